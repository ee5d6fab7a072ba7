// The unified-style binary index front (include/cphnsw/api/binary_index.hpp) on a small random
// sphere: a stored vector finds itself at Hamming distance 0, reranked results are exact, the packed
// codes agree with the component codes.  Modelled on the probe the reference's unified index passes
// (N = 2000, d = 128: a self query returns itself at distance 0).
#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

#include "cphnsw/api/binary_index.hpp"

using namespace cphnsw::binary;

static int failures = 0;
#define CHECK(c, what)                                  \
    do {                                                \
        if (!(c)) { std::printf("FAIL: %s\n", what); ++failures; } \
        else std::printf("ok:   %s\n", what);           \
    } while (0)

int main() {
    const size_t dim = 128, n = 2000;
    std::mt19937 rng(5);
    std::normal_distribution<float> g;
    std::vector<float> base(n * dim);
    for (size_t i = 0; i < n; ++i) {
        double s = 0;
        for (size_t d = 0; d < dim; ++d) { base[i * dim + d] = g(rng); s += double(base[i * dim + d]) * base[i * dim + d]; }
        for (size_t d = 0; d < dim; ++d) base[i * dim + d] /= float(std::sqrt(s));
    }
    BinaryCPHNSWIndex<64> index(IndexParams().set_dim(dim).set_M(32).set_ef_construction(200));
    CHECK(index.empty() && index.dim() == dim, "empty index");
    index.add_batch(base.data(), n - 10);
    for (size_t i = n - 10; i < n; ++i) index.add(base.data() + i * dim);
    CHECK(index.size() == n, "add_batch + add");
    size_t self0 = 0, exact = 0;
    for (size_t i = 0; i < 50; ++i) {
        auto r = index.search(base.data() + i * dim, SearchParams().set_k(5).set_ef(100).set_rerank(false));
        self0 += !r.empty() && r[0].distance == 0.0f;
        auto rr = index.search(base.data() + i * dim, SearchParams().set_k(5).set_ef(100).set_rerank(true, 50));
        exact += !rr.empty() && rr[0].id == i && std::fabs(rr[0].distance + 1.0f) < 1e-5f;
    }
    CHECK(self0 == 50, "a stored vector is found at Hamming distance 0");
    CHECK(exact == 50, "reranked self query returns itself with distance -1");
    auto w = index.codes();
    CHECK(w.size() == n * BinaryCPHNSWIndex<64>::NUM_WORDS, "packed codes: one 64-bit word per node");
    auto batch = index.search_batch(base.data(), 20, SearchParams().set_k(3));
    bool same = batch.size() == 20;
    for (size_t i = 0; same && i < 20; ++i) same &= batch[i] == index.search(base.data() + i * dim, SearchParams().set_k(3));
    CHECK(same, "search_batch equals search");
    {
        // residual codes: CPHNSWIndex<32, 16, 2> of the reference (K = 32 primary bits, R = 16, shift 2)
        BinaryCPHNSWIndex<32, 16, 2> res(IndexParams().set_dim(dim).set_M(16).set_ef_construction(200));
        res.add_batch(base.data(), n);
        auto rw = res.codes();
        BinaryCPHNSWIndex<32> prim(IndexParams().set_dim(dim).set_M(16).set_ef_construction(200));
        prim.add_batch(base.data(), 200);
        auto pw = prim.codes();
        bool same_primary = rw.size() == n;
        for (size_t i = 0; i < 200 && same_primary; ++i) same_primary = (rw[i] & 0xFFFFFFFFull) == pw[i] && (rw[i] >> 48) == 0;
        CHECK(same_primary, "residual index: bits 0..31 are the primary code of the K = 32 index, bits 32..47 the residual");
        size_t self = 0;
        for (size_t i = 0; i < 50; ++i) {
            auto r = res.search(base.data() + i * dim, SearchParams().set_k(5).set_ef(100).set_rerank(false));
            self += !r.empty() && r[0].distance == 0.0f;
            bool fits = true;
            for (auto& x : r) fits &= x.distance >= 0.f && x.distance <= float((32 << 2) + 16);
            self += fits ? 0 : 1000;
        }
        CHECK(self == 50, "residual index: self at combined distance 0, distances within (32 << 2) + 16");
    }
    std::printf("%s (%d failures)\n", failures ? "FAILED" : "ALL PASS", failures);
    return failures ? 1 : 0;
}
