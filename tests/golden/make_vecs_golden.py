"""Generates tests/golden/tiny.fvecs, tiny.ivecs and vecs_golden.npz.

The two small files are written in the fvecs / ivecs layout; vecs_golden.npz stores what the REFERENCE's own
readers return for them (load_fvecs / load_ivecs, evaluation/datasets/dataset_loader.hpp:40-108) and what its
normalize_vectors (:225-240) makes of the float rows.  Run where the reference checkout is available:

    make -C oracle ref REF=<reference checkout> && python tests/golden/make_vecs_golden.py
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.join(HERE, "..", "..")
sys.path.insert(0, os.path.join(ROOT, "sparse-text-kmeans_b200"))
from cphnsw_b200 import vecs_io  # noqa: E402


def main():
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libcphnsw_ref_scalar.so"))
    rng = np.random.default_rng(4242)
    x = (rng.standard_normal((9, 6)) * 4).astype(np.float32)
    x[1] = 0.0
    x[2, 0] = np.float32(-0.0)
    x[3] = 1e-30  # norm below the reference's 1e-10 threshold: left unchanged
    ids = rng.integers(0, 2**31, (4, 10), dtype=np.int64).astype(np.uint32)
    f, i = os.path.join(HERE, "tiny.fvecs"), os.path.join(HERE, "tiny.ivecs")
    vecs_io.write_fvecs(f, x)
    vecs_io.write_ivecs(i, ids)
    dim, count = C.c_uint64(), C.c_uint64()
    fx = np.zeros_like(x)
    assert ref.ref_load_fvecs(f.encode(), fx.ctypes.data_as(C.c_void_p), C.c_uint64(fx.size), C.byref(dim), C.byref(count)) == 0
    assert (dim.value, count.value) == x.shape[::-1]
    ix = np.zeros_like(ids)
    assert ref.ref_load_ivecs(i.encode(), ix.ctypes.data_as(C.c_void_p), C.c_uint64(ix.size), C.byref(dim), C.byref(count)) == 0
    fn = fx.copy()
    ref.ref_normalize_vectors(fn.ctypes.data_as(C.c_void_p), C.c_uint64(fn.shape[0]), C.c_uint64(fn.shape[1]))
    np.savez_compressed(os.path.join(HERE, "vecs_golden.npz"), fvecs=fx, ivecs=ix, fvecs_normalized=fn)
    print("wrote tiny.fvecs, tiny.ivecs, vecs_golden.npz")


if __name__ == "__main__":
    main()
