// The reference's own graph walk, SearchEngine<Policy>::search
// (include/cphnsw/search/search_engine.hpp:86-193), over a FlatGraph
// (include/cphnsw/graph/flat_graph.hpp) filled from a given adjacency and given packed sign-bit
// codes.  TEST INFRASTRUCTURE ONLY: it pins the control flow of the oracle's walk (and, through the
// oracle, the library's binary-code walk) to the one walk whose source survives in the reference.
//
// The three headers do not compile as shipped; the Makefile target `ref_search` compiles this file
// against a throw-away copy of the reference's include tree to which it applies three one-line
// fixes with sed (FlatGraph::new_query() made const, which search() needs on its `const Graph&`;
// the two-argument calls cphnsw::prefetch(p, 3) reduced to the one-argument function that
// core/memory.hpp:133 declares).  No patched copy is kept.  Scalar build only (with -mavx2 or
// -mavx512f the SIMD kernel headers redefine member templates of the scalar one).
#include <cstdint>
#include <cstring>
#include <vector>

#include "cphnsw/search/search_engine.hpp"

namespace {

using namespace cphnsw;

// W in full (k = ef), so that the pop-the-worst-first extraction at search_engine.hpp:181-190
// returns every member of W, ascending.
template <size_t K, size_t R, int Shift>
int run(const uint64_t* primary, const uint64_t* residual, uint64_t n, const uint32_t* adj, uint64_t M,
        const uint64_t* q_primary, const uint64_t* q_residual, uint64_t nq, const uint32_t* entry, uint64_t n_entry,
        uint64_t ef, uint32_t* out_ids, float* out_dist, uint32_t* out_count) {
    using Policy = UnifiedMetricPolicy<K, R, Shift>;
    using Code = typename Policy::CodeType;
    using Engine = SearchEngine<Policy>;
    auto make = [&](const uint64_t* p, const uint64_t* r, uint64_t i) {
        Code c;
        c.clear();
        for (size_t w = 0; w < Code::PRIMARY_WORDS; ++w) c.primary.signs[w] = p[i * Code::PRIMARY_WORDS + w];
        if constexpr (R > 0)
            for (size_t w = 0; w < Code::RESIDUAL_WORDS; ++w) c.residual.signs[w] = r[i * Code::RESIDUAL_WORDS + w];
        return c;
    };
    FlatGraph<Code> g(n, M);
    std::vector<Code> codes;
    for (uint64_t i = 0; i < n; ++i) {
        codes.push_back(make(primary, residual, i));
        g.add_node(codes.back());
    }
    for (uint64_t i = 0; i < n; ++i)
        for (uint64_t j = 0; j < M; ++j) {
            const uint32_t w = adj[i * M + j];
            if (w < n) g.add_neighbor(NodeId(i), w, codes[w], 0.0f);  // UnifiedNeighborBlock::add appends in order
        }
    const std::vector<NodeId> eps(entry, entry + n_entry);
    for (uint64_t q = 0; q < nq; ++q) {
        typename Policy::QueryType query;
        query.code = make(q_primary, q_residual, q);
        query.base = 0.0f;   // distance = base + scale * hamming (scalar_kernels.hpp:84-91)
        query.scale = 1.0f;
        query.query_norm = 1.0f;
        const std::vector<SearchResult> res = Engine::search(query, eps, ef, g, ef);
        out_count[q] = uint32_t(res.size());
        for (size_t t = 0; t < ef; ++t) {
            out_ids[q * ef + t] = t < res.size() ? res[t].id : 0xFFFFFFFFu;
            out_dist[q * ef + t] = t < res.size() ? res[t].distance : INFINITY;
        }
    }
    return 0;
}

}  // namespace

extern "C" {

// CPHNSWIndex<64, 0>: codes uint64[n] (bit r = sign bit of rotation r), queries uint64[nq].
int ref_search_64(const uint64_t* codes, uint64_t n, const uint32_t* adj, uint64_t M, const uint64_t* qcodes, uint64_t nq,
                  const uint32_t* entry, uint64_t n_entry, uint64_t ef, uint32_t* out_ids, float* out_dist,
                  uint32_t* out_count) {
    return run<64, 0, 0>(codes, nullptr, n, adj, M, qcodes, nullptr, nq, entry, n_entry, ef, out_ids, out_dist, out_count);
}

// CPHNSWIndex<32, 16, 2>: combined distance (h_primary << 2) + h_residual.
int ref_search_32_16_s2(const uint64_t* primary, const uint64_t* residual, uint64_t n, const uint32_t* adj, uint64_t M,
                        const uint64_t* q_primary, const uint64_t* q_residual, uint64_t nq, const uint32_t* entry,
                        uint64_t n_entry, uint64_t ef, uint32_t* out_ids, float* out_dist, uint32_t* out_count) {
    return run<32, 16, 2>(primary, residual, n, adj, M, q_primary, q_residual, nq, entry, n_entry, ef, out_ids, out_dist,
                          out_count);
}

}  // extern "C"
