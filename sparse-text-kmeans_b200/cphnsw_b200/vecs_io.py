"""fvecs / ivecs files (SIFT-1M / GIST-1M distribution format), read with the rules of the reference's
loaders (evaluation/datasets/dataset_loader.hpp:40-108): every record is a little-endian int32 length
followed by that many 4-byte values; the first record's length is the file's dimension, the record
count is file_size // record_size, later length fields are not checked."""
import os

import numpy as np


def _read(path, dtype, max_count):
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = np.fromfile(f, "<i4", 1)
        if head.size != 1 or head[0] <= 0:
            raise ValueError("not an fvecs/ivecs file (bad first length): %s" % path)
        dim = int(head[0])
        record = 4 + 4 * dim
        count = size // record
        if max_count:
            count = min(count, max_count)
        f.seek(0)
        raw = np.fromfile(f, "<u4", count * (dim + 1)).reshape(count, dim + 1)
    return np.ascontiguousarray(raw[:, 1:]).view(dtype)


def read_fvecs(path, max_count=0):
    """float32 [count][dim]."""
    return _read(path, np.float32, max_count)


def read_ivecs(path, max_count=0):
    """uint32 [count][k] (ground-truth neighbour ids)."""
    return _read(path, np.uint32, max_count)


def _write(path, a):
    a = np.ascontiguousarray(a)
    out = np.empty((a.shape[0], a.shape[1] + 1), "<u4")
    out[:, 0] = a.shape[1]
    out[:, 1:] = a.view("<u4")
    out.tofile(path)


def write_fvecs(path, a):
    _write(path, np.asarray(a, np.float32))


def write_ivecs(path, a):
    _write(path, np.asarray(a, np.uint32))


def normalize_rows(a):
    """Rows scaled to unit length like the reference's normalize_vectors (dataset_loader.hpp:225-240):
    fp32 accumulation in coordinate order, rows of norm <= 1e-10 left unchanged."""
    a = np.array(a, np.float32, copy=True)
    norm_sq = np.zeros(a.shape[0], np.float32)
    for d in range(a.shape[1]):
        norm_sq += a[:, d] * a[:, d]
    norm = np.sqrt(norm_sq)
    ok = norm > np.float32(1e-10)
    inv = np.ones_like(norm)
    inv[ok] = np.float32(1.0) / norm[ok]
    a *= inv[:, None]
    return a
