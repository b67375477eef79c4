"""Sequence preprocessing (keras/preprocessing/sequence.py)."""
import numpy as np


def pad_sequences(sequences, maxlen=None, dtype="int32", padding="pre", truncating="pre", value=0.0):
    """Lists of different lengths -> one [num_sequences, maxlen] array, padded / truncated at the front ('pre') or the back ('post')."""
    if padding not in ("pre", "post") or truncating not in ("pre", "post"):
        raise ValueError("padding and truncating are 'pre' or 'post'")
    lengths = [len(s) for s in sequences]
    maxlen = int(maxlen) if maxlen is not None else (max(lengths) if lengths else 0)
    out = np.full((len(sequences), maxlen), value, dtype=dtype)
    for i, s in enumerate(sequences):
        if not len(s) or maxlen == 0:
            continue
        t = list(s)[-maxlen:] if truncating == "pre" else list(s)[:maxlen]
        if padding == "post":
            out[i, :len(t)] = t
        else:
            out[i, maxlen - len(t):] = t
    return out
