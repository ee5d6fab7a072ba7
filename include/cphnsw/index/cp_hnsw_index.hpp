// CPHNSWIndex<ComponentT, K>: header-only C++ front of the cphnsw_b200 C ABI with the surface of the
// reference's legacy index class (its header is absent from the reference tree; the surface is the
// one its evaluation programs call — evaluation/eval_sift.cpp:228-283,387,430,
// evaluation/eval_master.cpp:89,145, evaluation/eval_main.cpp:42-43, evaluation/test_gpu_build.cpp:155-174,
// evaluation/debug_code_storage.cpp:75).  Host pointers in, results by value, ascending by distance;
// parameter errors throw std::invalid_argument like CPHNSWParams::finalize()
// (include/cphnsw/core/types.hpp:403-469); any other failure throws std::runtime_error.
//
// All arithmetic runs on the GPU behind the C ABI; this header holds no algorithm.
#pragma once

#include <array>
#include <cstddef>
#include <cstdint>
#include <limits>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include "../../cphnsw_b200.h"

namespace cphnsw {

using NodeId = uint32_t;                                                     // types.hpp:27
constexpr NodeId INVALID_NODE = std::numeric_limits<NodeId>::max();          // types.hpp:29
using Float = float;                                                         // types.hpp:41
using AsymmetricDist = float;                                                // types.hpp:38
using HammingDist = uint16_t;                                                // types.hpp:35

// One result of a k-NN search (types.hpp:347-362).
struct SearchResult {
    NodeId id;
    AsymmetricDist distance;
    bool operator<(const SearchResult& o) const { return distance < o.distance; }
    bool operator>(const SearchResult& o) const { return distance > o.distance; }
    bool operator==(const SearchResult& o) const { return id == o.id && distance == o.distance; }
};

// K-component cross-polytope code; component = (argmax index << 1) | negative (types.hpp:68-106).
// Only the components are stored by this implementation.
template <typename ComponentT, size_t K>
struct CPCode {
    std::array<ComponentT, K> components;
    static constexpr size_t decode_index(ComponentT c) { return c >> 1; }
    static constexpr bool decode_sign_negative(ComponentT c) { return c & 1; }
    static constexpr ComponentT encode(size_t index, bool is_negative) {
        return static_cast<ComponentT>((index << 1) | (is_negative ? 1 : 0));
    }
};

// Number of components in which two codes differ (the legacy hamming_distance(CPCode,CPCode);
// use sites evaluation/debug_estimator.cpp:149,172).  Trivial host helper for single pairs; batches
// go through CPHNSWIndex::code_distance.
template <typename ComponentT, size_t K>
inline HammingDist hamming_distance(const CPCode<ComponentT, K>& a, const CPCode<ComponentT, K>& b) {
    HammingDist d = 0;
    for (size_t r = 0; r < K; ++r) d += a.components[r] != b.components[r];
    return d;
}

// Index parameters (types.hpp:374-470).  `k` is the code width and must equal the template K.
struct CPHNSWParams {
    size_t dim = 0;
    size_t padded_dim = 0;
    size_t k = 32;
    size_t M = 32;
    size_t ef_construction = 200;
    bool keep_pruned = true;
    uint64_t seed = 42;
    size_t k_entry = 4;
    float rank_pruning_alpha = 1.1f;
    void finalize() {
        if (dim == 0) throw std::invalid_argument("CPHNSWParams: dim must be > 0");
        if (k == 0) throw std::invalid_argument("CPHNSWParams: k (code width) must be > 0");
        if (k > 256) throw std::invalid_argument("CPHNSWParams: k (code width) must be <= 256");
        if (M == 0) throw std::invalid_argument("CPHNSWParams: M (max connections) must be > 0");
        if (M > 64) throw std::invalid_argument("CPHNSWParams: M must be <= 64 (FLASH_MAX_M limit)");
        if (ef_construction < M) throw std::invalid_argument("CPHNSWParams: ef_construction must be >= M for good graph quality");
        if (ef_construction > 10000) throw std::invalid_argument("CPHNSWParams: ef_construction must be <= 10000");
        if (k_entry == 0) throw std::invalid_argument("CPHNSWParams: k_entry must be > 0");
        if (k_entry > 100) throw std::invalid_argument("CPHNSWParams: k_entry must be <= 100");
        if (rank_pruning_alpha < 1.0f) throw std::invalid_argument("CPHNSWParams: rank_pruning_alpha must be >= 1.0");
        if (rank_pruning_alpha > 3.0f) throw std::invalid_argument("CPHNSWParams: rank_pruning_alpha must be <= 3.0");
        padded_dim = 1;
        while (padded_dim < dim) padded_dim *= 2;
    }
};

template <typename ComponentT, size_t K>
class CPHNSWIndex {
    static_assert(std::is_same<ComponentT, uint8_t>::value || std::is_same<ComponentT, uint16_t>::value,
                  "ComponentT must be uint8_t or uint16_t");

public:
    using Code = CPCode<ComponentT, K>;

    // `device` >= 0 binds the index to that GPU; ALL_GPUS (the default) spreads it over every usable GPU of the box:
    // one replica per device, the bulk build sharded by row block, batched searches by query block, single-query
    // calls going round the replicas (cphnsw_b200_sharded_* in cphnsw_b200.h).  On a one-GPU box both are the same.
    static constexpr int ALL_GPUS = -1;
    CPHNSWIndex(size_t dim, size_t M = 32, size_t ef_construction = 200, uint64_t seed = 42,
                int fht_convention = CPHNSW_B200_FHT_AVX512, int device = ALL_GPUS) {
        create(dim, M, ef_construction, seed, fht_convention, device);
    }
    explicit CPHNSWIndex(const CPHNSWParams& p, int fht_convention = CPHNSW_B200_FHT_AVX512, int device = ALL_GPUS) {
        if (p.k != K) throw std::invalid_argument("CPHNSWParams: k must equal the index's code width K");
        create(p.dim, p.M, p.ef_construction, p.seed, fht_convention, device);
        set_param("keep_pruned", p.keep_pruned ? 1.0 : 0.0);
        set_param("k_entry", double(p.k_entry));
        set_param("rank_pruning_alpha", double(p.rank_pruning_alpha));
    }
    ~CPHNSWIndex() { cphnsw_b200_sharded_destroy(s_); }
    CPHNSWIndex(const CPHNSWIndex&) = delete;
    CPHNSWIndex& operator=(const CPHNSWIndex&) = delete;
    CPHNSWIndex(CPHNSWIndex&& o) noexcept : s_(o.s_), h_(o.h_) { o.s_ = nullptr, o.h_ = nullptr; }

    // ---- index file (the reference has no save/load) ---------------------------------------------
    void save(const std::string& path) const { check(cphnsw_b200_save(h_, path.c_str())); }
    static CPHNSWIndex load(const std::string& path, int device = ALL_GPUS) {
        cphnsw_b200_sharded* s = nullptr;
        check(cphnsw_b200_sharded_load(path.c_str(), device < 0 ? 0 : 1, device < 0 ? nullptr : &device, &s));
        cphnsw_b200_index* h = cphnsw_b200_sharded_replica(s, 0);
        double k = 0, cb = 0;
        cphnsw_b200_get_param(h, "K", &k);
        cphnsw_b200_get_param(h, "component_bytes", &cb);
        if (size_t(k) != K || size_t(cb) != sizeof(ComponentT)) {
            cphnsw_b200_sharded_destroy(s);
            throw std::invalid_argument("index file holds another code type than this CPHNSWIndex<ComponentT,K>");
        }
        return CPHNSWIndex(s, Adopt{});
    }

    // replica 0: every read-only call and every stage call of this class goes to it
    cphnsw_b200_index* handle() const { return h_; }
    cphnsw_b200_sharded* sharded() const { return s_; }
    int gpus() const { return cphnsw_b200_sharded_gpus(s_); }
    void set_param(const char* name, double v) { check(cphnsw_b200_sharded_set_param(s_, name, v)); }
    size_t dim() const { return cphnsw_b200_dim(h_); }
    size_t padded_dim() const { return cphnsw_b200_padded_dim(h_); }
    size_t size() const { return cphnsw_b200_size(h_); }

    // ---- construction -------------------------------------------------------------------------
    // add / add_batch insert into the existing graph (new links + reverse links); add_batch_parallel
    // rebuilds the graph over everything added so far.  On an empty index all three are the bulk build.
    NodeId add(const Float* vec) {
        NodeId id = NodeId(size());
        add_batch(vec, 1);
        return id;
    }
    void add_batch(const Float* vecs, size_t n) { check(cphnsw_b200_sharded_add_batch(s_, vecs, n)); }
    void add_batch_parallel(const Float* vecs, size_t n) { check(cphnsw_b200_sharded_add_batch_parallel(s_, vecs, n)); }
    // build_with_gpu_knn (evaluation/test_gpu_build.cpp:168-174): bulk build from a k-candidate kNN graph
    // (CP-code distance).  prune = true prunes it by rank with the detour threshold alpha, the CAGRA graph
    // optimisation the parameter is documented for (types.hpp:399-400; rule in cphnsw_b200.h at
    // cphnsw_b200_rank_prune); prune = false keeps the M nearest candidates.  add_batch_parallel is the
    // build that prunes with select_neighbors (the HNSW heuristic).
    void build_with_gpu_knn(const Float* vecs, size_t n, size_t k = 64, bool prune = true, float alpha = 1.1f) {
        if (!(alpha >= 1.0f) || alpha > 3.0f) throw std::invalid_argument("build_with_gpu_knn: alpha must be in [1.0, 3.0]");
        if (k == 0 || k > 64) throw std::invalid_argument("build_with_gpu_knn: k must be in 1..64");
        if (size() != 0) throw std::invalid_argument("build_with_gpu_knn: the index must be empty");
        const char* names[4] = {"knn_k", "prune", "rank_prune", "rank_pruning_alpha"};
        const double want[4] = {double(k), 1.0, prune ? 1.0 : 0.0, double(alpha)};
        double old[4] = {0, 1, 0, 1.1};
        for (int i = 0; i < 4; ++i) check(cphnsw_b200_get_param(h_, names[i], &old[i]));
        int rc = 0;
        for (int i = 0; i < 4 && rc == 0; ++i) rc = cphnsw_b200_sharded_set_param(s_, names[i], want[i]);
        if (rc == 0 && !prune) rc = cphnsw_b200_sharded_set_param(s_, "prune", 0.0);
        if (rc == 0) rc = cphnsw_b200_sharded_add_batch_parallel(s_, vecs, n);
        // last_error() belongs to the failing call: restore the tunables only after reading it
        std::string msg = rc ? cphnsw_b200_last_error() : "";
        for (int i = 0; i < 4; ++i) cphnsw_b200_sharded_set_param(s_, names[i], old[i]);
        if (rc) fail(rc, msg);
    }

    // ---- search ---------------------------------------------------------------------------------
    std::vector<SearchResult> search(const Float* q, size_t k, size_t ef) const {
        return search_batch(q, 1, k, ef)[0];
    }
    std::vector<SearchResult> search_and_rerank(const Float* q, size_t k, size_t ef, size_t rerank_k) const {
        return search_and_rerank_batch(q, 1, k, ef, rerank_k)[0];
    }
    std::vector<std::vector<SearchResult>> search_batch(const Float* q, size_t nq, size_t k, size_t ef) const {
        std::vector<uint32_t> ids(nq * k);
        std::vector<float> d(nq * k);
        check(cphnsw_b200_sharded_search(s_, 0, q, nq, uint32_t(k), uint32_t(ef), 0, ids.data(), d.data(), nullptr));
        return unpack(ids, d, nq, k);
    }
    std::vector<std::vector<SearchResult>> search_and_rerank_batch(const Float* q, size_t nq, size_t k, size_t ef,
                                                                   size_t rerank_k) const {
        std::vector<uint32_t> ids(nq * k);
        std::vector<float> d(nq * k);
        check(cphnsw_b200_sharded_search(s_, 1, q, nq, uint32_t(k), uint32_t(ef), uint32_t(rerank_k), ids.data(), d.data(),
                                         nullptr));
        return unpack(ids, d, nq, k);
    }

    std::vector<SearchResult> search_multiprobe(const Float* q, size_t k, size_t ef, size_t num_probes) const {
        return search_multiprobe_batch(q, 1, k, ef, num_probes)[0];
    }
    std::vector<std::vector<SearchResult>> search_multiprobe_batch(const Float* q, size_t nq, size_t k, size_t ef,
                                                                   size_t num_probes) const {
        std::vector<uint32_t> ids(nq * k);
        std::vector<float> d(nq * k);
        check(cphnsw_b200_sharded_search(s_, 2, q, nq, uint32_t(k), uint32_t(ef), uint32_t(num_probes), ids.data(), d.data(),
                                         nullptr));
        return unpack(ids, d, nq, k);
    }

    // ---- diagnostics (evaluation/eval_sift.cpp:266-283, evaluation/eval_main.cpp:52,128-189) -------
    struct Calibration {  // exact distance ~ alpha * CP score + beta over sampled node pairs
        float alpha = 1.0f, beta = 0.0f, r_squared = 0.0f;
        size_t num_samples = 0;
    };
    std::vector<SearchResult> brute_force_search(const Float* q, size_t k) const {
        std::vector<uint32_t> ids(k);
        std::vector<float> d(k);
        check(cphnsw_b200_sharded_search(s_, 3, q, 1, uint32_t(k), uint32_t(k), 0, ids.data(), d.data(), nullptr));
        return unpack(ids, d, 1, k)[0];
    }
    size_t verify_connectivity() const {
        uint64_t r = 0;
        check(cphnsw_b200_verify_connectivity(h_, &r));
        return size_t(r);
    }
    Calibration calibrate(size_t num_samples = 1000, uint64_t seed = 42) {
        // the fit is kept in the handle: every replica computes it (same samples, same result)
        for (int g = 0; g < gpus(); ++g)
            check(cphnsw_b200_calibrate(cphnsw_b200_sharded_replica(s_, g), num_samples, seed, nullptr, nullptr, nullptr));
        return get_calibration();
    }
    Calibration get_calibration() const {
        double a = 1, b = 0, r = 0;
        uint64_t m = 0;
        check(cphnsw_b200_get_calibration(h_, &a, &b, &r, &m));
        Calibration c;
        c.alpha = float(a), c.beta = float(b), c.r_squared = float(r), c.num_samples = size_t(m);
        return c;
    }
    std::vector<SearchResult> search_calibrated(const Float* q, size_t k, size_t ef) const {
        return search_calibrated_and_rerank(q, k, ef, 0);
    }
    std::vector<SearchResult> search_calibrated_and_rerank(const Float* q, size_t k, size_t ef, size_t rerank_k) const {
        std::vector<uint32_t> ids(k);
        std::vector<float> d(k);
        check(cphnsw_b200_sharded_search(s_, 4, q, 1, uint32_t(k), uint32_t(ef), uint32_t(rerank_k), ids.data(), d.data(), nullptr));
        return unpack(ids, d, 1, k)[0];
    }

    // ---- stages ---------------------------------------------------------------------------------
    std::vector<Code> encode(const Float* vecs, size_t n) const {
        std::vector<Code> out(n);
        static_assert(sizeof(Code) == K * sizeof(ComponentT), "CPCode must be a plain component array");
        check(cphnsw_b200_encode(h_, vecs, n, out.data()));
        return out;
    }
    Code get_code(NodeId id) const {
        if (id >= size()) throw std::out_of_range("get_code: node id out of range");
        Code c;
        check(cphnsw_b200_get_code(h_, id, &c));
        return c;
    }
    std::vector<HammingDist> code_distance(const std::vector<Code>& a, const std::vector<Code>& b) const {
        std::vector<HammingDist> out(a.size() * b.size());
        check(cphnsw_b200_code_distance(h_, a.data(), a.size(), b.data(), b.size(), out.data()));
        return out;
    }
    std::vector<NodeId> adjacency() const {
        std::vector<NodeId> adj(size() * size_t(param("M")));
        check(cphnsw_b200_get_adjacency(h_, adj.data()));
        return adj;
    }
    double param(const char* name) const {
        double v = 0;
        check(cphnsw_b200_get_param(h_, name, &v));
        return v;
    }

private:
    struct Adopt {};
    CPHNSWIndex(cphnsw_b200_sharded* s, Adopt) : s_(s), h_(cphnsw_b200_sharded_replica(s, 0)) {}
    void create(size_t dim, size_t M, size_t ef_construction, uint64_t seed, int fht_convention, int device) {
        check(cphnsw_b200_sharded_create(dim, uint32_t(K), uint32_t(sizeof(ComponentT)), uint32_t(M), uint32_t(ef_construction),
                                         seed, fht_convention, 0, device < 0 ? 0 : 1, device < 0 ? nullptr : &device, &s_));
        h_ = cphnsw_b200_sharded_replica(s_, 0);
    }
    cphnsw_b200_sharded* s_ = nullptr;  // owns the replicas
    cphnsw_b200_index* h_ = nullptr;    // replica 0

    static void fail(int rc, const std::string& msg) {
        if (rc == CPHNSW_B200_E_INVALID) throw std::invalid_argument(msg);
        throw std::runtime_error(msg);
    }
    static void check(int rc) {
        if (rc != 0) fail(rc, cphnsw_b200_last_error());
    }
    static std::vector<std::vector<SearchResult>> unpack(const std::vector<uint32_t>& ids, const std::vector<float>& d,
                                                         size_t nq, size_t k) {
        std::vector<std::vector<SearchResult>> out(nq);
        for (size_t q = 0; q < nq; ++q)
            for (size_t t = 0; t < k; ++t)
                if (ids[q * k + t] != INVALID_NODE) out[q].push_back({ids[q * k + t], d[q * k + t]});
        return out;
    }
};

using CPHNSWIndex8 = CPHNSWIndex<uint8_t, 16>;    // evaluation/eval_main.cpp:42
using CPHNSWIndex32 = CPHNSWIndex<uint8_t, 32>;   // evaluation/test_tiered.cpp:58
using CPHNSWIndex16 = CPHNSWIndex<uint16_t, 16>;

}  // namespace cphnsw
