// cphnsw::cuda::GPUEncoder<ComponentT, K> and cphnsw::cuda::GPUBruteForce with the interface of the
// reference's classes of the same names (include/cphnsw/cuda/gpu_encoder.cuh:24-93 and :101-156), on
// the B200 library.  Header-only and plain C++ (no CUDA headers needed): every method is one call
// of the C ABI in cphnsw_b200.h.  Errors throw (std::invalid_argument for parameter violations,
// std::runtime_error otherwise); nothing exits the process.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>

#include "cphnsw_b200.h"

namespace cphnsw {

using Float = float;  // include/cphnsw/core/types.hpp:41

namespace cuda {

namespace detail {
inline void check(int rc) {
    if (rc == 0) return;
    const std::string msg = cphnsw_b200_last_error();
    if (rc == CPHNSW_B200_E_INVALID) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}
}  // namespace detail

// Codes equal those of the reference's CPU encoder built with AVX-512 (the default); pass
// CPHNSW_B200_FHT_SCALAR for the butterfly order of the reference's own CUDA kernels
// (src/cuda/gpu_encoder.cu:75-125).
template <typename ComponentT, size_t K>
class GPUEncoder {
    static_assert(sizeof(ComponentT) == 1 || sizeof(ComponentT) == 2, "ComponentT is uint8_t or uint16_t");

public:
    GPUEncoder(size_t dim, uint64_t seed = 42, int fht_convention = CPHNSW_B200_FHT_AVX512, int device = 0)
        : dim_(dim), seed_(seed), convention_(fht_convention), device_(device) {
        detail::check(cphnsw_b200_create(dim, uint32_t(K), uint32_t(sizeof(ComponentT)), 1, 1, seed, fht_convention, device, &h_));
        padded_dim_ = size_t(cphnsw_b200_padded_dim(h_));
    }
    ~GPUEncoder() {
        cphnsw_b200_destroy(h_);
        cphnsw_b200_destroy(hp_);
    }
    GPUEncoder(const GPUEncoder&) = delete;
    GPUEncoder& operator=(const GPUEncoder&) = delete;
    GPUEncoder(GPUEncoder&& o) noexcept { *this = std::move(o); }
    GPUEncoder& operator=(GPUEncoder&& o) noexcept {
        if (this != &o) {
            cphnsw_b200_destroy(h_);
            cphnsw_b200_destroy(hp_);
            h_ = o.h_, hp_ = o.hp_, dim_ = o.dim_, padded_dim_ = o.padded_dim_, seed_ = o.seed_;
            convention_ = o.convention_, device_ = o.device_;
            o.h_ = o.hp_ = nullptr;
        }
        return *this;
    }

    // h_vectors [num_vecs x dim] -> h_codes [num_vecs x K]   (gpu_encoder.cuh:45-52)
    void encode_batch(const Float* h_vectors, size_t num_vecs, ComponentT* h_codes) {
        detail::check(cphnsw_b200_encode(h_, h_vectors, num_vecs, h_codes));
    }

    // d_vectors [num_vecs x padded_dim] on the device, zero padded -> d_codes [num_vecs x K] on the
    // device   (gpu_encoder.cuh:54-61).  The sign tables depend on the padded dimension only, so a
    // second handle of dimension padded_dim yields the same codes.
    void encode_batch_device(const Float* d_vectors, size_t num_vecs, ComponentT* d_codes) {
        if (!hp_)
            detail::check(cphnsw_b200_create(padded_dim_, uint32_t(K), uint32_t(sizeof(ComponentT)), 1, 1, seed_, convention_,
                                             device_, &hp_));
        detail::check(cphnsw_b200_encode_dev(hp_, d_vectors, num_vecs, d_codes, nullptr, nullptr, nullptr));
    }

    // codes and magnitudes |x_argmax| per rotation for queries   (gpu_encoder.cuh:63-72)
    void encode_queries_batch(const Float* h_vectors, size_t num_queries, ComponentT* h_codes, Float* h_magnitudes) {
        detail::check(cphnsw_b200_encode_queries(h_, h_vectors, num_queries, h_codes, nullptr, h_magnitudes));
    }

    size_t dim() const { return dim_; }
    size_t padded_dim() const { return padded_dim_; }
    cphnsw_b200_index* handle() const { return h_; }

private:
    cphnsw_b200_index* h_ = nullptr;
    cphnsw_b200_index* hp_ = nullptr;  // dimension padded_dim, made on the first encode_batch_device
    size_t dim_ = 0, padded_dim_ = 0;
    uint64_t seed_ = 42;
    int convention_ = CPHNSW_B200_FHT_AVX512, device_ = 0;
};

// Exact search and rerank by -<q,x> (the reference multiplies with cuBLAS; here the dot product is
// accumulated in fp32 in d order, so results equal a plain CPU loop; ties go to the lower id).
class GPUBruteForce {
public:
    GPUBruteForce(size_t dim, size_t num_base, int device = 0) : dim_(dim), num_base_(num_base) {
        // the handle only carries the dimension and the vectors; its code parameters are not used
        detail::check(cphnsw_b200_create(dim, 1, 2, 1, 1, 42, CPHNSW_B200_FHT_AVX512, device, &h_));
    }
    ~GPUBruteForce() { cphnsw_b200_destroy(h_); }
    GPUBruteForce(const GPUBruteForce&) = delete;
    GPUBruteForce& operator=(const GPUBruteForce&) = delete;

    // gpu_encoder.cuh:110-113
    void set_base_vectors(const Float* h_base, size_t num_base) {
        detail::check(cphnsw_b200_set_exact_base(h_, h_base, num_base));
        num_base_ = num_base;
    }

    // gpu_encoder.cuh:115-125; k <= 128; h_distances = -<q,x>, ascending
    void search(const Float* h_queries, size_t num_queries, size_t k, uint32_t* h_indices, Float* h_distances) {
        detail::check(cphnsw_b200_exact_search_batch(h_, h_queries, num_queries, uint32_t(k), h_indices, h_distances));
    }

    // gpu_encoder.cuh:127-140
    void rerank(const Float* h_queries, const uint32_t* h_candidate_ids, size_t num_queries, size_t num_candidates, size_t k,
                uint32_t* h_indices, Float* h_distances) {
        detail::check(cphnsw_b200_rerank_batch(h_, h_queries, num_queries, h_candidate_ids, uint32_t(num_candidates), uint32_t(k),
                                               h_indices, h_distances));
    }

    size_t dim() const { return dim_; }
    size_t num_base() const { return num_base_; }

private:
    cphnsw_b200_index* h_ = nullptr;
    size_t dim_ = 0, num_base_ = 0;
};

}  // namespace cuda
}  // namespace cphnsw
