// cphnsw::binary::BinaryCPHNSWIndex<K>: the reference's unified index CPHNSWIndex<K, 0> (sign-bit
// codes, Hamming metric; include/cphnsw/api/index.hpp:60-260, include/cphnsw/api/config.hpp:17-100)
// on the B200 library.  Same parameter structs and method names; header-only, holds no algorithm.
// BinaryCPHNSWIndex<K, R, Shift> is CPHNSWIndex<K, R, Shift>: R residual bits, combined distance
// (h_primary << Shift) + h_residual (include/cphnsw/core/types.hpp:284-302); K + R <= 128.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "cphnsw_b200.h"

namespace cphnsw {
namespace binary {

using NodeId = uint32_t;

struct SearchResult {  // include/cphnsw/core/types.hpp:40-52
    NodeId id;
    float distance;
    bool operator<(const SearchResult& o) const { return distance < o.distance; }
    bool operator==(const SearchResult& o) const { return id == o.id && distance == o.distance; }
};

struct IndexParams {  // config.hpp:17-45
    size_t dim = 0, M = 32, ef_construction = 200;
    uint64_t seed = 42;
    size_t initial_capacity = 1024;  // accepted for source compatibility; device buffers grow on demand
    IndexParams& set_dim(size_t d) { dim = d; return *this; }
    IndexParams& set_M(size_t m) { M = m; return *this; }
    IndexParams& set_ef_construction(size_t ef) { ef_construction = ef; return *this; }
    IndexParams& set_seed(uint64_t s) { seed = s; return *this; }
    IndexParams& set_capacity(size_t c) { initial_capacity = c; return *this; }
};

struct BuildParams {  // config.hpp:47-68; the build always runs on the GPU of the handle
    size_t num_threads = 0;
    bool use_gpu = true;
    int gpu_device = 0;
    size_t gpu_tile_size = 16384;
    bool verbose = false;
    BuildParams& set_threads(size_t n) { num_threads = n; return *this; }
    BuildParams& set_gpu(bool use, int device = 0) { use_gpu = use; gpu_device = device; return *this; }
    BuildParams& set_verbose(bool v) { verbose = v; return *this; }
};

struct SearchParams {  // config.hpp:74-100
    size_t k = 10, ef = 100, num_entry_points = 1;
    bool rerank = true;
    size_t rerank_k = 200;
    SearchParams& set_k(size_t n) { k = n; return *this; }
    SearchParams& set_ef(size_t e) { ef = e; return *this; }
    SearchParams& set_rerank(bool r, size_t rk = 200) { rerank = r; rerank_k = rk; return *this; }
};

template <size_t K, size_t R = 0, int Shift = 2>
class BinaryCPHNSWIndex {
    static_assert(K >= 1 && K <= 256, "1 <= K <= 256 sign bits");
    static_assert(R == 0 || (K % 4 == 0 && K + R <= 128 && Shift >= 0 && Shift <= 4),
                  "residual codes: K a multiple of 4, K + R <= 128, 0 <= Shift <= 4");

public:
    // words per node returned by codes(): bits 0..K-1 primary, K..K+R-1 residual (BinaryCodeStorage, codes.hpp:24)
    static constexpr size_t NUM_WORDS = (K + R + 63) / 64;

    explicit BinaryCPHNSWIndex(const IndexParams& p, int device = 0) : params_(p) {
        check(cphnsw_b200_create_binary(p.dim, uint32_t(K + R), uint32_t(p.M), uint32_t(p.ef_construction), p.seed,
                                        CPHNSW_B200_FHT_AVX512, device, &h_));
        if (R) {
            check(cphnsw_b200_set_param(h_, "residual_bits", double(R)));
            check(cphnsw_b200_set_param(h_, "residual_shift", double(Shift)));
        }
    }
    explicit BinaryCPHNSWIndex(size_t dim) : BinaryCPHNSWIndex(IndexParams().set_dim(dim)) {}
    ~BinaryCPHNSWIndex() { cphnsw_b200_destroy(h_); }
    BinaryCPHNSWIndex(const BinaryCPHNSWIndex&) = delete;
    BinaryCPHNSWIndex& operator=(const BinaryCPHNSWIndex&) = delete;

    // add (index.hpp:98-120) and add_batch (index.hpp:125-164): incremental insertion; the first batch
    // on an empty index is built in bulk
    NodeId add(const float* vec) {
        const NodeId id = NodeId(size());
        check(cphnsw_b200_add_batch(h_, vec, 1));
        return id;
    }
    void add_batch(const float* vecs, size_t n, const BuildParams& = BuildParams()) { check(cphnsw_b200_add_batch(h_, vecs, n)); }

    // search (index.hpp:177-214): walk under the Hamming distance to the query's code with beam
    // max(ef, k); with params.rerank the best rerank_k are re-scored exactly (here with -<q,x>,
    // the reference uses the squared L2 distance: the same order for unit vectors)
    std::vector<SearchResult> search(const float* query, const SearchParams& p = SearchParams()) const {
        return search_batch(query, 1, p)[0];
    }
    std::vector<SearchResult> search(const float* query, size_t k) const { return search(query, SearchParams().set_k(k)); }
    std::vector<std::vector<SearchResult>> search_batch(const float* queries, size_t nq,
                                                        const SearchParams& p = SearchParams()) const {
        std::vector<uint32_t> ids(nq * p.k);
        std::vector<float> d(nq * p.k);
        const size_t rr = p.rerank ? (p.rerank_k > p.k ? p.rerank_k : p.k) : 0;
        if (rr)
            check(cphnsw_b200_search_and_rerank_batch(h_, queries, nq, uint32_t(p.k), uint32_t(p.ef), uint32_t(rr), ids.data(),
                                                      d.data(), nullptr));
        else
            check(cphnsw_b200_search_batch(h_, queries, nq, uint32_t(p.k), uint32_t(p.ef), ids.data(), d.data(), nullptr));
        std::vector<std::vector<SearchResult>> out(nq);
        for (size_t q = 0; q < nq; ++q)
            for (size_t t = 0; t < p.k; ++t)
                if (ids[q * p.k + t] != CPHNSW_B200_INVALID_NODE) out[q].push_back({ids[q * p.k + t], d[q * p.k + t]});
        return out;
    }

    // the packed codes, NUM_WORDS uint64 per node (ResidualCode<K,R>: primary bits, then residual bits)
    std::vector<uint64_t> codes() const {
        std::vector<uint64_t> w(size() * NUM_WORDS);
        check(cphnsw_b200_get_binary_codes(h_, w.data()));
        return w;
    }

    size_t size() const { return cphnsw_b200_size(h_); }
    bool empty() const { return size() == 0; }
    size_t dim() const { return params_.dim; }
    const IndexParams& params() const { return params_; }
    cphnsw_b200_index* handle() const { return h_; }

private:
    IndexParams params_;
    cphnsw_b200_index* h_ = nullptr;

    static void check(int rc) {
        if (rc == 0) return;
        const std::string msg = cphnsw_b200_last_error();
        if (rc == CPHNSW_B200_E_INVALID) throw std::invalid_argument(msg);
        throw std::runtime_error(msg);
    }
};

}  // namespace binary
}  // namespace cphnsw
