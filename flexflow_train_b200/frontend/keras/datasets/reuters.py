"""Reuters newswire topics from a local ``reuters.npz`` (object arrays x, y of word-index lists and labels)."""
import os

import numpy as np


def load_data(path="reuters.npz", num_words=None, skip_top=0, maxlen=None, test_split=0.2, seed=113, start_char=1, oov_char=2,
              index_from=3):
    """((x_train, y_train), (x_test, y_test)) with Keras's conventions: indices shifted by `index_from`, `start_char` in
    front, words outside [skip_top, num_words) replaced by `oov_char`, the last `test_split` of a seeded shuffle held out."""
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} not found: place Keras's reuters.npz there (data sets are not downloaded)")
    with np.load(path, allow_pickle=True) as f:
        xs, labels = list(f["x"]), np.asarray(f["y"])
    order = np.random.RandomState(seed).permutation(len(xs))
    xs, labels = [xs[i] for i in order], labels[order]
    xs = [[start_char] + [w + index_from for w in x] for x in xs]
    if maxlen:
        keep = [i for i, x in enumerate(xs) if len(x) < maxlen]
        xs, labels = [xs[i] for i in keep], labels[keep]
    hi = num_words or (max(max(x) for x in xs) + 1 if xs else 0)
    xs = [[w if skip_top <= w < hi else oov_char for w in x] for x in xs]
    cut = int(len(xs) * (1 - test_split))
    as_obj = lambda rows: np.array(rows, dtype=object)  # noqa: E731
    return (as_obj(xs[:cut]), labels[:cut]), (as_obj(xs[cut:]), labels[cut:])
