"""Shared helpers of the test-suite."""
import hashlib

import numpy as np


def digest(*arrays):
    """SHA-256 of int64 little-endian bytes of the concatenated arrays (the golden file's rule)."""
    cat = np.concatenate([np.asarray(a).astype("<i8").ravel() for a in arrays])
    return hashlib.sha256(cat.tobytes()).hexdigest()


def rel_err(a, b):
    """Max-norm relative error ||a-b||_inf / ||b||_inf, the measure the parity gates use."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    denom = np.abs(b).max()
    return float(np.abs(a - b).max() / (denom if denom > 0 else 1.0))


def fully_connected_blocks(batch, length):
    """The graph of graph_kernel/test.py:79-136: `batch` independent fully connected graphs of
    `length` nodes; edge id enumerates (graph, src, dst) row-major."""
    b = np.arange(batch)[:, None, None]
    s = np.arange(length)[None, :, None]
    d = np.arange(length)[None, None, :]
    src = (b * length + s + 0 * d).ravel().astype(np.int64)
    dst = (b * length + d + 0 * s).ravel().astype(np.int64)
    return src, dst, batch * length
