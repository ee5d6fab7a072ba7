// Property checks of CPHNSWIndex<ComponentT,K> through the C++ header, modelled on the reference's
// QA protocol (evaluation/qa_protocol.cpp): identity queries, ordering, duplicates, zero vector,
// tiny inputs, parameter validation, stored code == fresh code, recall non-decreasing in ef.
// Prints one line per check and exits non-zero on the first failure.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <random>
#include <set>
#include <vector>

#include "cphnsw/index/cp_hnsw_index.hpp"

using namespace cphnsw;

static int failures = 0;
#define CHECK(cond, name)                                       \
    do {                                                        \
        bool ok__ = (cond);                                     \
        std::printf("[%s] %s\n", ok__ ? "PASS" : "FAIL", name); \
        if (!ok__) ++failures;                                  \
    } while (0)

static std::vector<float> unit_vectors(size_t n, size_t dim, uint64_t seed) {
    std::mt19937_64 rng(seed);
    std::normal_distribution<float> g(0.f, 1.f);
    std::vector<float> v(n * dim);
    for (size_t i = 0; i < n; ++i) {
        float s = 0;
        for (size_t d = 0; d < dim; ++d) {
            v[i * dim + d] = g(rng);
            s += v[i * dim + d] * v[i * dim + d];
        }
        s = std::sqrt(s);
        for (size_t d = 0; d < dim; ++d) v[i * dim + d] /= s;
    }
    return v;
}

int main() {
    const size_t dim = 128, n = 5000;
    auto base = unit_vectors(n, dim, 42);

    // parameter validation (types.hpp:403-469)
    {
        bool threw = false;
        try { CPHNSWIndex<uint8_t, 32> bad(0); } catch (const std::invalid_argument&) { threw = true; }
        CHECK(threw, "dim == 0 throws invalid_argument");
        threw = false;
        try { CPHNSWIndex<uint8_t, 32> bad(128, 65, 200); } catch (const std::invalid_argument&) { threw = true; }
        CHECK(threw, "M > 64 throws invalid_argument");
        threw = false;
        try { CPHNSWIndex<uint8_t, 32> bad(256); } catch (const std::invalid_argument&) { threw = true; }
        CHECK(threw, "uint8_t components with padded dim 256 throw");
        CPHNSWParams p;
        p.dim = 128; p.k = 32; p.k_entry = 0;
        threw = false;
        try { p.finalize(); } catch (const std::invalid_argument&) { threw = true; }
        CHECK(threw, "CPHNSWParams::finalize rejects k_entry == 0");
    }

    CPHNSWIndex<uint8_t, 32> index(dim, 32, 200);
    index.set_param("entry_scan", 256);
    index.add_batch_parallel(base.data(), n);
    CHECK(index.size() == n, "size() after add_batch_parallel");

    // identity: a stored vector finds itself first, with a negative distance (qa_protocol.cpp:65-114)
    {
        size_t hits = 0, negative = 0;
        for (size_t i = 0; i < 100; ++i) {
            auto r = index.search_and_rerank(base.data() + i * dim, 10, 100, 200);
            hits += !r.empty() && r[0].id == i;
            negative += !r.empty() && r[0].distance < 0;
        }
        CHECK(hits == 100 && negative == 100, "identity query returns own id with negative distance");
    }
    // ordering (qa_protocol.cpp:116-166)
    {
        bool asc = true, neg = true;
        for (size_t i = 0; i < 50; ++i) {
            auto r = index.search(base.data() + i * dim, 10, 100);
            for (size_t t = 1; t < r.size(); ++t) asc &= r[t - 1].distance <= r[t].distance;
            neg &= !r.empty() && r[0].distance < 0;
        }
        CHECK(asc && neg, "results ascend and start negative");
    }
    // stored code == fresh code (debug_code_storage.cpp:63-105)
    {
        auto fresh = index.encode(base.data(), 64);
        bool same = true;
        for (NodeId i = 0; i < 64; i += 7) same &= hamming_distance(index.get_code(i), fresh[i]) == 0;
        CHECK(same, "stored code equals a fresh encode (distance 0)");
    }
    // batch distance agrees with the pairwise helper
    {
        auto codes = index.encode(base.data(), 40);
        std::vector<CPCode<uint8_t, 32>> a(codes.begin(), codes.begin() + 8), b(codes.begin() + 8, codes.end());
        auto d = index.code_distance(a, b);
        bool same = true;
        for (size_t i = 0; i < a.size(); ++i)
            for (size_t j = 0; j < b.size(); ++j) same &= d[i * b.size() + j] == hamming_distance(a[i], b[j]);
        CHECK(same, "batched code distance equals pairwise count of differing components");
    }
    // adjacency validity: ids in range, no self loops (debug_gpu_knn.cpp:42-68)
    {
        auto adj = index.adjacency();
        bool ok = true;
        for (size_t i = 0; i < n; ++i)
            for (size_t t = 0; t < 32; ++t) {
                NodeId v = adj[i * 32 + t];
                ok &= (v == INVALID_NODE) || (v < n && v != i);
            }
        CHECK(ok, "adjacency ids in range and no self loops");
    }
    // recall non-decreasing in ef (qa_protocol.cpp:559-640), measured against a brute-force top-10
    {
        auto q = unit_vectors(50, dim, 7);
        double last = -1;
        bool mono = true;
        for (size_t ef : {10, 50, 200, 800}) {
            auto res = index.search_and_rerank_batch(q.data(), 50, 10, ef, ef < 10 ? 10 : ef);
            size_t hit = 0;
            for (size_t qi = 0; qi < 50; ++qi) {
                std::vector<std::pair<float, NodeId>> all(n);
                for (size_t i = 0; i < n; ++i) {
                    float dot = 0;
                    for (size_t d = 0; d < dim; ++d) dot += q[qi * dim + d] * base[i * dim + d];
                    all[i] = {-dot, NodeId(i)};
                }
                std::partial_sort(all.begin(), all.begin() + 10, all.end());
                std::set<NodeId> gt;
                for (size_t t = 0; t < 10; ++t) gt.insert(all[t].second);
                for (auto& r : res[qi]) hit += gt.count(r.id);
            }
            double recall = hit / 500.0;
            mono &= recall >= last - 1e-9;
            last = recall;
        }
        CHECK(mono && last > 0.3, "recall non-decreasing in ef");
    }
    // search_multiprobe (evaluation/eval_sift.cpp:430): ascending integer code distances, one probe equals
    // a plain walk under the code distance, more probes can only lower the best distance
    {
        auto q = unit_vectors(20, dim, 11);
        auto one = index.search_multiprobe_batch(q.data(), 20, 10, 100, 1);
        auto many = index.search_multiprobe_batch(q.data(), 20, 10, 100, 16);
        bool ok = true;
        for (size_t qi = 0; qi < 20; ++qi) {
            ok &= one[qi].size() == 10 && many[qi].size() == 10;
            for (size_t t = 1; t < many[qi].size(); ++t) ok &= many[qi][t - 1].distance <= many[qi][t].distance;
            for (auto& r : many[qi]) ok &= r.distance >= 0 && r.distance <= 32 && r.distance == std::floor(r.distance);
            ok &= many[qi][0].distance <= one[qi][0].distance;
        }
        CHECK(ok, "search_multiprobe returns ascending code distances and improves with probes");
    }
    // diagnostics: connectivity (eval_main.cpp:52), brute force by CP score (eval_sift.cpp:283),
    // calibration sign (qa_protocol.cpp:263-282) and calibrated search (eval_main.cpp:170-189)
    {
        const size_t reach = index.verify_connectivity();
        CHECK(reach > n * 9 / 10 && reach <= n, "verify_connectivity reaches (nearly) every node");
        auto bf = index.brute_force_search(base.data() + 7 * dim, 10);
        bool asc = bf.size() == 10 && bf[0].id == 7;
        for (size_t t = 1; t < bf.size(); ++t) asc &= bf[t - 1].distance <= bf[t].distance;
        CHECK(asc, "brute_force_search finds the stored vector first, ascending scores");
        auto calib = index.calibrate(1000);
        CHECK(calib.alpha > 0 && calib.r_squared > 0.3f && calib.num_samples == 1000, "calibrate: alpha > 0 (positive correlation)");
        auto plain = index.search(base.data() + 7 * dim, 10, 100);
        auto cal = index.search_calibrated(base.data() + 7 * dim, 10, 100);
        bool same = plain.size() == cal.size();
        for (size_t t = 0; same && t < plain.size(); ++t)
            same &= plain[t].id == cal[t].id && std::fabs(cal[t].distance - (calib.alpha * plain[t].distance + calib.beta)) < 1e-4f;
        CHECK(same, "search_calibrated returns the ids of search with distances alpha * score + beta");
        CHECK(cal[0].distance < -0.5f, "calibrated distance of a stored vector to itself is near -1");
        auto rr = index.search_and_rerank(base.data() + 7 * dim, 10, 100, 50);
        auto crr = index.search_calibrated_and_rerank(base.data() + 7 * dim, 10, 100, 50);
        bool eq = rr.size() == crr.size();
        for (size_t t = 0; eq && t < rr.size(); ++t) eq &= rr[t] == crr[t];
        CHECK(eq, "search_calibrated_and_rerank equals search_and_rerank");
    }
    // index file: a loaded index answers like the one that was saved
    {
        const std::string path = "/tmp/cphnsw_b200_qa_index.bin";
        index.save(path);
        auto copy = CPHNSWIndex<uint8_t, 32>::load(path);
        auto q = unit_vectors(5, dim, 99);
        auto r1 = index.search_and_rerank_batch(q.data(), 5, 10, 100, 50);
        auto r2 = copy.search_and_rerank_batch(q.data(), 5, 10, 100, 50);
        CHECK(copy.size() == n && r1 == r2, "load(save(index)) returns the same results");
        bool threw = false;
        try { auto wrong = CPHNSWIndex<uint16_t, 16>::load(path); } catch (const std::invalid_argument&) { threw = true; }
        CHECK(threw, "loading into another CPHNSWIndex<ComponentT,K> throws");
        std::remove(path.c_str());
    }
    // edge cases (qa_protocol.cpp:409-553): tiny index, duplicates, zero vector
    {
        CPHNSWIndex<uint8_t, 32> tiny(dim, 32, 200);
        std::vector<float> v(5 * dim, 0.f);
        for (size_t i = 1; i < 5; ++i) v[i * dim + (i % 2)] = 1.f;  // vector 0 is all-zero, 1==3, 2==4
        tiny.add_batch(v.data(), 5);
        auto r = tiny.search_and_rerank(v.data() + dim, 3, 10, 5);
        bool finite = true;
        for (auto& x : r) finite &= std::isfinite(x.distance);
        CHECK(tiny.size() == 5 && r.size() == 3 && finite, "tiny index with duplicates and a zero vector");
        CHECK(r[0].id == 1 && r[1].id == 3, "duplicates tie-break by id");
    }
    {
        CPHNSWIndex<uint16_t, 16> wide(300, 16, 200);
        auto b = unit_vectors(500, 300, 3);
        wide.add_batch_parallel(b.data(), 500);
        auto r = wide.search_and_rerank(b.data(), 5, 50, 50);
        CHECK(!r.empty() && r[0].id == 0, "uint16_t components, padded dim 512");
    }
    {
        // build_with_gpu_knn (evaluation/test_gpu_build.cpp:168-174): k candidates per node, pruned by rank with the
        // detour threshold alpha = the bulk build with knn_k = k, rank_prune = 1 and that alpha
        auto b = unit_vectors(3000, dim, 11);
        CPHNSWIndex<uint8_t, 32> g(dim, 32, 200), ref(dim, 32, 200), cut(dim, 32, 200);
        g.build_with_gpu_knn(b.data(), 3000, 64, true, 1.1f);
        ref.set_param("knn_k", 64);
        ref.set_param("rank_prune", 1);
        ref.set_param("rank_pruning_alpha", 1.1);
        ref.add_batch_parallel(b.data(), 3000);
        bool same = g.size() == 3000 && g.adjacency() == ref.adjacency() && g.param("rank_prune") == 0.0;
        for (size_t q = 0; q < 20 && same; ++q) {
            auto x = g.search_and_rerank(b.data() + q * dim, 5, 50, 50), y = ref.search_and_rerank(b.data() + q * dim, 5, 50, 50);
            same = x.size() == y.size();
            for (size_t t = 0; t < x.size() && same; ++t) same = x[t] == y[t];
        }
        CHECK(same, "build_with_gpu_knn(k=64, prune, alpha) is the bulk build with rank-based pruning");
        CHECK(g.verify_connectivity() > 2900, "build_with_gpu_knn graph is connected from the entry nodes");
        cut.build_with_gpu_knn(b.data(), 3000, 64, false, 1.1f);
        auto r = cut.search_and_rerank(b.data() + 7 * dim, 5, 50, 50);
        CHECK(cut.size() == 3000 && !r.empty() && r[0].id == 7, "build_with_gpu_knn without pruning");
        bool threw = false;
        try { cut.build_with_gpu_knn(b.data(), 10, 64, true, 0.5f); } catch (const std::invalid_argument&) { threw = true; }
        CHECK(threw, "build_with_gpu_knn rejects alpha < 1");
    }
    std::printf("%s (%d failures)\n", failures ? "FAILED" : "ALL PASS", failures);
    return failures ? 1 : 0;
}
