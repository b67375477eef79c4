"""CIFAR-10 from a local directory holding the python-version batches (data_batch_1..5, test_batch)."""
import os
import pickle

import numpy as np


def load_batch(fpath, label_key="labels"):
    with open(fpath, "rb") as f:
        d = pickle.load(f, encoding="bytes")
    d = {(k.decode("utf8") if isinstance(k, bytes) else k): v for k, v in d.items()}
    data = np.asarray(d["data"]).reshape(-1, 3, 32, 32)
    return data, np.asarray(d[label_key])


def load_data(path="cifar-10-batches-py", num_samples=50000):
    """((x_train, y_train), (x_test, y_test)), images uint8 [N, 3, 32, 32] (channels first, as the legacy loader), labels [N, 1]."""
    if not os.path.isdir(path):
        raise FileNotFoundError(f"{path} not found: unpack cifar-10-python.tar.gz there (data sets are not downloaded)")
    xs, ys = [], []
    for i in range(1, 6):
        x, y = load_batch(os.path.join(path, f"data_batch_{i}"))
        xs.append(x)
        ys.append(y)
    x_train, y_train = np.concatenate(xs)[:num_samples], np.concatenate(ys)[:num_samples]
    x_test, y_test = load_batch(os.path.join(path, "test_batch"))
    return (x_train, y_train.reshape(-1, 1)), (x_test, y_test.reshape(-1, 1))
