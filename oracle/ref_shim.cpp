// Thin extern "C" wrapper around the REFERENCE project's own hot-path headers, compiled in
// place from the reference checkout (-I <reference>/include).  TEST INFRASTRUCTURE ONLY.
//
// Nothing from the reference is copied here: this file only instantiates and calls the
// reference's classes so that the oracle restatement (cphnsw_oracle.cpp) and the golden
// fixtures can be validated against the real thing.  The Makefile builds it three times
// (no -m flags, -mavx2, -mavx512f), because the reference's FHT picks its code path from the
// compiler's ISA macros (include/cphnsw/encoder/transform/fht.hpp:7-17) and the three builds
// produce three different sign conventions.
//
// The resulting libraries live in oracle/_ref/ and exist only where the reference checkout
// is available at build time.

#include <cstdint>
#include <cstring>
#include <vector>

#include "cphnsw/core/types.hpp"
#include "cphnsw/encoder/cp_encoder.hpp"
#include "cphnsw/encoder/rotation.hpp"
#include "cphnsw/encoder/transform/fht.hpp"
#ifdef CPHNSW_REF_EVAL_DIR
// the reference's dataset readers (evaluation/datasets/dataset_loader.hpp), included in place
#include "datasets/dataset_loader.hpp"
// the unified distance kernels compile in the scalar build only
#include "cphnsw/distance/metric_policy.hpp"
#endif

extern "C" {

// 0 = scalar build, 1 = AVX2 build, 2 = AVX-512 build (fht.hpp:207-215 dispatch).
int ref_convention() {
#if CPHNSW_FHT_AVX512
    return 2;
#elif CPHNSW_FHT_AVX2
    return 1;
#else
    return 0;
#endif
}

int ref_fht(float* v, uint64_t n) {
    cphnsw::fht(v, n);
    return 0;
}

int ref_fht_scalar(float* v, uint64_t n) {
    cphnsw::fht_scalar(v, n);
    return 0;
}

// int8 [K][3][P], rotation r seeded seed + r as RotationChain does (rotation.hpp:173-178).
int ref_sign_tables(uint64_t dim, uint64_t K, uint64_t seed, int8_t* out) {
    for (uint64_t r = 0; r < K; ++r) {
        cphnsw::RandomHadamardRotation rot(dim, seed + r);
        size_t P = rot.padded_dim();
        const auto& s = rot.get_signs();
        for (int l = 0; l < 3; ++l) std::memcpy(out + (r * 3 + l) * P, s[l].data(), P);
    }
    return 0;
}

int ref_argmax_abs(const float* v, uint64_t n, uint64_t* idx, float* mag) {
    size_t i;
    float m;
    cphnsw::detail::find_argmax_abs(v, n, i, m);
    *idx = i;
    *mag = m;
    return 0;
}

// K-component code from reference parts: RandomHadamardRotation::apply_copy (rotation.hpp:104-111),
// detail::find_argmax_abs (cp_encoder.hpp:25-92), sign test of cp_encoder.hpp:174,
// CPCode::encode (types.hpp:88-90).  Optional rotated [n][K][P] and magnitudes [n][K].
int ref_encode(const float* x, uint64_t n, uint64_t dim, uint64_t K, uint64_t comp_bytes,
               uint64_t seed, void* codes, float* rotated, float* magnitudes) {
    std::vector<cphnsw::RandomHadamardRotation> rots;
    for (uint64_t r = 0; r < K; ++r) rots.emplace_back(dim, seed + r);
    size_t P = rots[0].padded_dim();
    std::vector<float> buf(P);
    for (uint64_t i = 0; i < n; ++i)
        for (uint64_t r = 0; r < K; ++r) {
            rots[r].apply_copy(x + i * dim, buf.data());
            size_t idx;
            float mag;
            cphnsw::detail::find_argmax_abs(buf.data(), P, idx, mag);
            bool neg = buf[idx] < 0;
            if (comp_bytes == 1)
                ((uint8_t*)codes)[i * K + r] = cphnsw::CPCode<uint8_t, 1>::encode(idx, neg);
            else
                ((uint16_t*)codes)[i * K + r] = cphnsw::CPCode<uint16_t, 1>::encode(idx, neg);
            if (rotated) std::memcpy(rotated + (i * K + r) * P, buf.data(), P * sizeof(float));
            if (magnitudes) magnitudes[i * K + r] = mag;
        }
    return 0;
}

// The reference's shipped encoder, unmodified: CPEncoder<32,0>::encode_batch
// (cp_encoder.hpp:244-260).  Emits the 32 primary sign bits of each vector; it does the same
// K x 3 FHTs + argmax per vector as the K-byte encode, so it is the timed CPU reference for
// the encode stage and a cross-check of the sign bit of every component.
int ref_encode_batch_signbits32(const float* x, uint64_t n, uint64_t dim, uint64_t seed, uint32_t* out) {
    cphnsw::CPEncoder<32, 0> enc(dim, seed);
    std::vector<cphnsw::ResidualCode<32, 0>> codes(n);
    enc.encode_batch(x, n, codes.data());
    for (uint64_t i = 0; i < n; ++i) out[i] = (uint32_t)codes[i].primary.signs[0];
    return 0;
}

// The unified encoder with 64 sign bits, and the reference's own Hamming distance between two of
// its primary codes (include/cphnsw/distance/detail/scalar_kernels.hpp:37-47).
int ref_encode_batch_signbits64(const float* x, uint64_t n, uint64_t dim, uint64_t seed, uint64_t* out) {
    cphnsw::CPEncoder<64, 0> enc(dim, seed);
    std::vector<cphnsw::ResidualCode<64, 0>> codes(n);
    enc.encode_batch(x, n, codes.data());
    for (uint64_t i = 0; i < n; ++i) out[i] = codes[i].primary.signs[0];
    return 0;
}

// The unified encoder with residual bits, CPEncoder<32, 16> (include/cphnsw/encoder/cp_encoder.hpp:161-184,282-300)
int ref_encode_batch_residual_32_16(const float* x, uint64_t n, uint64_t dim, uint64_t seed, uint64_t* primary,
                                    uint64_t* residual) {
    // one vector at a time through encode(): the reference's encode_batch runs encode_residual on a
    // buffer shared by all OpenMP threads (cp_encoder.hpp:286-300), so its residual bits are only
    // defined single-threaded
    cphnsw::CPEncoder<32, 16> enc(dim, seed);
    for (uint64_t i = 0; i < n; ++i) {
        const cphnsw::ResidualCode<32, 16> c = enc.encode(x + i * dim);
        primary[i] = c.primary.signs[0];
        residual[i] = c.residual.signs[0];
    }
    return 0;
}

}  // extern "C"

#ifdef CPHNSW_REF_EVAL_DIR
extern "C" {

// the reference's combined distance (primary << 2) + residual
// (include/cphnsw/distance/detail/scalar_kernels.hpp:57-76)
int ref_hamming_combined_32_16_s2(const uint64_t* pa, const uint64_t* ra, uint64_t na, const uint64_t* pb, const uint64_t* rb,
                                  uint64_t nb, uint32_t* out) {
    for (uint64_t i = 0; i < na; ++i)
        for (uint64_t j = 0; j < nb; ++j) {
            cphnsw::ResidualCode<32, 16> a, b;
            a.clear(), b.clear();
            a.primary.signs[0] = pa[i], a.residual.signs[0] = ra[i];
            b.primary.signs[0] = pb[j], b.residual.signs[0] = rb[j];
            out[i * nb + j] = cphnsw::detail::hamming_combined_scalar<32, 16, 2>(a, b);
        }
    return 0;
}

int ref_hamming64(const uint64_t* a, uint64_t na, const uint64_t* b, uint64_t nb, uint32_t* out) {
    for (uint64_t i = 0; i < na; ++i)
        for (uint64_t j = 0; j < nb; ++j) {
            cphnsw::BinaryCodeStorage<64> ca, cb;
            ca.signs[0] = a[i];
            cb.signs[0] = b[j];
            out[i * nb + j] = cphnsw::detail::hamming_primary_scalar<64>(ca, cb);
        }
    return 0;
}

// the reference's load_fvecs / load_ivecs / normalize_vectors; out may be null to query the shape
int ref_load_fvecs(const char* path, float* out, uint64_t cap, uint64_t* dim, uint64_t* count) {
    try {
        size_t d = 0, c = 0;
        auto v = cphnsw::eval::load_fvecs(path, d, c);
        *dim = d, *count = c;
        if (out && v.size() <= cap) std::memcpy(out, v.data(), v.size() * sizeof(float));
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

int ref_load_ivecs(const char* path, uint32_t* out, uint64_t cap, uint64_t* k, uint64_t* count) {
    try {
        size_t kk = 0, c = 0;
        auto v = cphnsw::eval::load_ivecs(path, kk, c);
        *k = kk, *count = c;
        if (out && kk * c <= cap)
            for (size_t i = 0; i < c; ++i) std::memcpy(out + i * kk, v[i].data(), kk * sizeof(uint32_t));
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

int ref_normalize_vectors(float* v, uint64_t count, uint64_t dim) {
    cphnsw::eval::normalize_vectors(v, count, dim);
    return 0;
}

}  // extern "C"
#endif
