"""Generates tests/golden/residual_golden.npz from the REFERENCE's unified sources with residual bits.

For seeded inputs: the primary (32 bits) and residual (16 bits) words of the reference's
CPEncoder<32,16> (include/cphnsw/encoder/cp_encoder.hpp:161-184,282-300; scalar, AVX2 and AVX-512
builds of its headers; one vector at a time through encode(), because its encode_batch shares the
residual buffer between OpenMP threads) and the combined distances its hamming_combined_scalar<32,16,2> gives between
them (include/cphnsw/distance/detail/scalar_kernels.hpp:57-76).  Run where the reference checkout is
available:

    make -C oracle ref REF=<reference checkout> && python tests/golden/make_residual_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import oracle as O  # noqa: E402


def main():
    rng = np.random.default_rng(3216)
    out = {}
    for dim in (128, 100, 24):
        x = rng.standard_normal((40, dim)).astype(np.float32)
        x[1] = 0.0
        x[3] = x[0]
        x[5] = -x[4]
        out["x_%d" % dim] = x
        for conv in (O.FHT_SCALAR, O.FHT_AVX2, O.FHT_AVX512):
            p, r = O.Ref(conv).encode_batch_residual_32_16(x, 42)
            out["primary_%d_c%d" % (dim, conv)] = p
            out["residual_%d_c%d" % (dim, conv)] = r
    p, r = out["primary_128_c2"], out["residual_128_c2"]
    out["combined_128_c2"] = O.Ref(O.FHT_SCALAR).hamming_combined_32_16_s2(p[:16], r[:16], p, r)
    np.savez_compressed(os.path.join(HERE, "residual_golden.npz"), **out)
    print("wrote residual_golden.npz")


if __name__ == "__main__":
    main()
