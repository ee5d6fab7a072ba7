"""Generates tests/golden/binary_golden.npz from the REFERENCE's unified (binary-code) sources.

For seeded inputs: the packed 64-bit sign codes of the reference's CPEncoder<64,0> (scalar, AVX2 and
AVX-512 builds of its headers) and the Hamming distances its hamming_primary_scalar<64> gives between
them (include/cphnsw/distance/detail/scalar_kernels.hpp:37-47).  Run where the reference checkout is
available:

    make -C oracle ref REF=<reference checkout> && python tests/golden/make_binary_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import oracle as O  # noqa: E402


def main():
    rng = np.random.default_rng(64064)
    out = {}
    for dim in (128, 96, 20):
        x = rng.standard_normal((48, dim)).astype(np.float32)
        x[1] = 0.0
        x[3] = x[0]
        out["x_%d" % dim] = x
        for conv in (O.FHT_SCALAR, O.FHT_AVX2, O.FHT_AVX512):
            out["bits_%d_c%d" % (dim, conv)] = O.Ref(conv).encode_batch_signbits64(x, 42)
    b = out["bits_128_c2"]
    out["hamming_128_c2"] = O.Ref(O.FHT_SCALAR).hamming64(b[:20], b)
    np.savez_compressed(os.path.join(HERE, "binary_golden.npz"), **out)
    print("wrote binary_golden.npz")


if __name__ == "__main__":
    main()
