"""Generates tests/golden/encode_golden.npz from the REFERENCE's own headers.

Run where the reference checkout is available (it is compiled in place by ``make -C oracle ref``):

    make -C oracle ref REF=<reference checkout> && python tests/golden/make_golden.py

For each FHT build convention (scalar / AVX2 / AVX-512 builds of the reference's headers) the
fixture stores, for a set of seeded inputs: the reference's FHT outputs, its sign tables, its
K-component codes, and for two small cases its rotated vectors and winning magnitudes.
The inputs are stored alongside, so the fixture is self-contained.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import oracle as O  # noqa: E402

CASES = [  # (dim, K, component_bytes, n)
    (5, 4, 1, 12), (8, 4, 1, 12), (16, 4, 1, 12), (33, 8, 1, 12), (96, 32, 1, 24), (128, 32, 1, 24),
    (128, 16, 2, 8), (200, 8, 2, 8), (960, 8, 2, 6),
]


def main():
    out = {}
    rng = np.random.default_rng(20240)
    for n in (1, 2, 4, 8, 16, 32, 64, 128, 256, 1024):
        out["fht_in_%d" % n] = rng.standard_normal(n).astype(np.float32)
    out["fht_in_4"] = np.array([1, 2, 3, 4], np.float32)  # tests/unit/test_hadamard.cpp:26-47
    for ci, (dim, K, cb, n) in enumerate(CASES):
        x = rng.standard_normal((n, dim)).astype(np.float32)
        x[1] = 0.0                      # zero vector
        x[2] = np.abs(x[2])             # non-negative
        x[3] = x[0]                     # duplicate
        if dim >= 8:
            x[4] = 0.0
            x[4, :2] = (1.0, -1.0)      # exact ties in magnitude
        out["x_%d" % ci] = x
    for conv in (O.FHT_SCALAR, O.FHT_AVX2, O.FHT_AVX512):
        R = O.Ref(conv)
        for n in (1, 2, 4, 8, 16, 32, 64, 128, 256, 1024):
            out["fht_%d_c%d" % (n, conv)] = R.fht(out["fht_in_%d" % n])
        for ci, (dim, K, cb, n) in enumerate(CASES):
            x = out["x_%d" % ci]
            if conv == 0:
                out["signs_%d" % ci] = np.packbits(R.sign_tables(dim, K, 42) > 0)
            want_rot = dim in (16, 128) and cb == 1
            if want_rot:
                codes, rot, mag = R.encode(x[:4], K, cb, 42, True)
                out["rot_%d_c%d" % (ci, conv)] = rot
                out["mag_%d_c%d" % (ci, conv)] = mag
            out["codes_%d_c%d" % (ci, conv)] = R.encode(x, K, cb, 42)
    out["cases"] = np.array(CASES, np.int64)
    np.savez_compressed(os.path.join(HERE, "encode_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "encode_golden.npz"), os.path.getsize(os.path.join(HERE, "encode_golden.npz")), "bytes")


if __name__ == "__main__":
    main()
