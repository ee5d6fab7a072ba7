"""The CPU oracle against fixtures produced by the reference's own headers (tests/golden/make_golden.py)
and against the reference's known-answer tests (tests/unit/test_hadamard.cpp)."""
import os

import numpy as np
import pytest

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "encode_golden.npz"))
CASES = [tuple(int(v) for v in row) for row in GOLD["cases"]]
CONVS = (0, 1, 2)


def unpack_signs(ci, dim, K, oracle):
    P = oracle.next_pow2(dim)
    bits = np.unpackbits(GOLD["signs_%d" % ci])[: K * 3 * P].reshape(K, 3, P)
    return np.where(bits > 0, 1, -1).astype(np.int8)


def test_fht_known_answer(oracle):
    # H4 * [1,2,3,4] = [10,-2,-4,0]  (tests/unit/test_hadamard.cpp:26-47; pins the scalar convention)
    assert oracle.fht(np.array([1, 2, 3, 4], np.float32), 0).tolist() == [10.0, -2.0, -4.0, 0.0]


@pytest.mark.parametrize("n", [8, 16, 32, 64, 128, 256])
def test_fht_self_inverse_and_norm(oracle, n):
    # FHT(FHT(x)) = n x and |FHT(x)| = sqrt(n) |x|  (test_hadamard.cpp:11-23, 50-76)
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32)
    for conv in CONVS:
        y = oracle.fht(x, conv)
        # the SIMD conventions differ from the scalar one by a +-1 diagonal, so |.| and norms agree
        assert np.allclose(np.linalg.norm(y), np.linalg.norm(x) * np.sqrt(n), rtol=1e-4)
    y = oracle.fht(oracle.fht(x, 0), 0)
    assert np.allclose(y, n * x, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("conv", CONVS)
@pytest.mark.parametrize("n", [1, 2, 4, 8, 16, 32, 64, 128, 256, 1024])
def test_fht_matches_reference_build(oracle, conv, n):
    got = oracle.fht(GOLD["fht_in_%d" % n], conv)
    assert np.array_equal(got.view(np.uint32), GOLD["fht_%d_c%d" % (n, conv)].view(np.uint32))


@pytest.mark.parametrize("ci", range(len(CASES)))
def test_sign_tables_match_reference(oracle, ci):
    dim, K, cb, n = CASES[ci]
    assert np.array_equal(oracle.sign_tables(dim, K, 42), unpack_signs(ci, dim, K, oracle))


@pytest.mark.parametrize("conv", CONVS)
@pytest.mark.parametrize("ci", range(len(CASES)))
def test_codes_match_reference(oracle, conv, ci):
    dim, K, cb, n = CASES[ci]
    signs = unpack_signs(ci, dim, K, oracle)
    x = GOLD["x_%d" % ci]
    codes = oracle.encode(x, K, cb, signs, conv)
    assert np.array_equal(codes, GOLD["codes_%d_c%d" % (ci, conv)])
    key = "rot_%d_c%d" % (ci, conv)
    if key in GOLD:
        c, rot, mag = oracle.encode(x[:4], K, cb, signs, conv, want_rotated=True)
        assert np.array_equal(rot.view(np.uint32) & 0x7FFFFFFF, GOLD[key].view(np.uint32) & 0x7FFFFFFF)
        nz = GOLD[key] != 0  # -0.0 and +0.0 are the same value to every consumer
        assert np.array_equal(rot[nz], GOLD[key][nz])
        assert np.array_equal(mag, GOLD["mag_%d_c%d" % (ci, conv)])


@pytest.mark.parametrize("conv", CONVS)
def test_live_reference_when_available(oracle, conv):
    """Where the reference's headers were compiled here (oracle/_ref), compare on fresh inputs too."""
    if not oracle.ref_available(conv):
        pytest.skip("reference shim not built on this machine")
    R = oracle.Ref(conv)
    rng = np.random.default_rng(7 + conv)
    for dim, K, cb in ((128, 32, 1), (96, 32, 1), (960, 4, 2), (20, 8, 1)):
        x = rng.standard_normal((40, dim)).astype(np.float32)
        signs = oracle.sign_tables(dim, K, 42)
        assert np.array_equal(signs, R.sign_tables(dim, K, 42))
        assert np.array_equal(oracle.encode(x, K, cb, signs, conv), R.encode(x, K, cb, 42))
    x = rng.standard_normal((64, 128)).astype(np.float32)
    codes = oracle.encode(x, 32, 1, oracle.sign_tables(128, 32, 42), conv)
    bits = ((codes & 1).astype(np.uint64) << np.arange(32, dtype=np.uint64)).sum(axis=1).astype(np.uint32)
    # the reference's shipped encoder keeps exactly the sign bit of each component
    assert np.array_equal(bits, R.encode_batch_signbits32(x, 42))


BIN = np.load(os.path.join(os.path.dirname(__file__), "golden", "binary_golden.npz"))


def pack64(codes):
    return ((codes & 1).astype(np.uint64) << np.arange(64, dtype=np.uint64)).sum(axis=1).astype(np.uint64)


@pytest.mark.parametrize("conv", CONVS)
@pytest.mark.parametrize("dim", [128, 96, 20])
def test_sign_bits_are_the_unified_encoders_code(oracle, dim, conv):
    """Bit 0 of every component = the primary binary code of the reference's unified encoder
    (CPEncoder<64,0>, include/cphnsw/encoder/cp_encoder.hpp:161-184), for every FHT build."""
    x = BIN["x_%d" % dim]
    codes = oracle.encode(x, 64, 1 if dim <= 128 else 2, oracle.sign_tables(dim, 64, 42), conv)
    assert np.array_equal(pack64(codes), BIN["bits_%d_c%d" % (dim, conv)])


def test_component_mismatch_of_sign_codes_is_the_unified_hamming_distance(oracle):
    """code_distance on sign-only components = hamming_primary_scalar<64> of the packed codes
    (include/cphnsw/distance/detail/scalar_kernels.hpp:37-47)."""
    x = BIN["x_128"]
    codes = (oracle.encode(x, 64, 1, oracle.sign_tables(128, 64, 42), 2) & 1).astype(np.uint8)
    assert np.array_equal(oracle.code_distance(codes[:20], codes), BIN["hamming_128_c2"].astype(np.uint16))


RES = np.load(os.path.join(os.path.dirname(__file__), "golden", "residual_golden.npz"))


def pack_bits(codes, first, count):
    return ((codes[:, first:first + count] & 1).astype(np.uint64) << np.arange(count, dtype=np.uint64)).sum(axis=1).astype(np.uint64)


@pytest.mark.parametrize("conv", CONVS)
@pytest.mark.parametrize("dim", [128, 100, 24])
def test_residual_bits_are_rotations_K_onwards(oracle, dim, conv):
    """CPEncoder<32,16> (include/cphnsw/encoder/cp_encoder.hpp:161-184,282-300): the residual chain is
    seeded seed + K, so its bits are the sign bits of rotations 32..47 of one chain of 48."""
    x = RES["x_%d" % dim]
    codes = oracle.encode(x, 48, 1, oracle.sign_tables(dim, 48, 42), conv)
    assert np.array_equal(pack_bits(codes, 0, 32), RES["primary_%d_c%d" % (dim, conv)])
    assert np.array_equal(pack_bits(codes, 32, 16), RES["residual_%d_c%d" % (dim, conv)])


def test_weighted_code_distance_is_the_combined_hamming_distance(oracle):
    """(h_primary << 2) + h_residual = hamming_combined_scalar<32,16,2>
    (include/cphnsw/distance/detail/scalar_kernels.hpp:57-76)."""
    x = RES["x_128"]
    codes = (oracle.encode(x, 48, 1, oracle.sign_tables(128, 48, 42), 2) & 1).astype(np.uint8)
    with oracle.residual_weighting(32, 2):
        d = oracle.code_distance(codes[:16], codes)
    assert np.array_equal(d.astype(np.uint32), RES["combined_128_c2"])
    # the setting does not outlive the block
    plain = (codes[:16, None, :] != codes[None, :, :]).sum(axis=2)
    assert np.array_equal(oracle.code_distance(codes[:16], codes), plain)

