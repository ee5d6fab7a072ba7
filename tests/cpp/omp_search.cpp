// Searches from an OpenMP loop, one query per call, the way the reference's evaluation programs drive
// the index (evaluation/eval_sift.cpp:279-283 brute_force_search, :380-387 search, :423-430 and
// :462-469 search_multiprobe, :531 search + rerank): every thread calls the const search methods of one
// shared CPHNSWIndex.  Each result must equal what the batch call returns for that query.
// Prints one line per check and exits non-zero on the first failure.
#include <omp.h>

#include <cmath>
#include <cstdio>
#include <random>
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

static std::vector<float> clustered(size_t n, size_t dim, size_t clusters, uint64_t seed) {
    std::mt19937_64 rng(seed);
    std::normal_distribution<float> g(0.f, 1.f);
    std::vector<float> centres(clusters * dim), v(n * dim);
    for (auto& c : centres) c = g(rng);
    for (size_t i = 0; i < n; ++i) {
        const size_t c = rng() % clusters;
        float s = 0;
        for (size_t d = 0; d < dim; ++d) {
            v[i * dim + d] = centres[c * dim + d] + 0.3f * g(rng);
            s += v[i * dim + d] * v[i * dim + d];
        }
        s = std::sqrt(s);
        for (size_t d = 0; d < dim; ++d) v[i * dim + d] /= s;
    }
    return v;
}

static bool same(const std::vector<SearchResult>& a, const std::vector<SearchResult>& b) {
    if (a.size() != b.size()) return false;
    for (size_t i = 0; i < a.size(); ++i)
        if (!(a[i] == b[i])) return false;
    return true;
}

int main() {
    const size_t dim = 128, n = 20000, nq = 192, k = 10;
    const auto base = clustered(n, dim, 40, 1);
    const auto queries = clustered(nq, dim, 40, 2);
    CPHNSWParams p;
    p.dim = dim;
    p.k = 32;
    p.k_entry = 8;
    p.finalize();
    CPHNSWIndex<uint8_t, 32> idx(p);
    idx.set_param("entry_scan", 512);
    idx.add_batch_parallel(base.data(), n);
    const CPHNSWIndex<uint8_t, 32>& index = idx;  // the search methods are const, as in the reference

    const auto want_search = index.search_batch(queries.data(), nq, k, 100);
    const auto want_rerank = index.search_and_rerank_batch(queries.data(), nq, k, 100, 200);
    const auto want_probe = index.search_multiprobe_batch(queries.data(), nq, k, 64, 4);

    omp_set_num_threads(16);
    std::vector<std::vector<SearchResult>> got_search(nq), got_rerank(nq), got_probe(nq), got_brute(nq);
    int errors = 0;
#pragma omp parallel for schedule(dynamic) reduction(+ : errors)
    for (size_t q = 0; q < nq; ++q) {
        try {
            const float* query = queries.data() + q * dim;
            got_search[q] = index.search(query, k, 100);
            got_rerank[q] = index.search_and_rerank(query, k, 100, 200);
            got_probe[q] = index.search_multiprobe(query, k, 64, 4);
            if (q % 16 == 0) got_brute[q] = index.brute_force_search(query, k);
        } catch (const std::exception& e) {
            std::printf("thread %d: %s\n", omp_get_thread_num(), e.what());
            ++errors;
        }
    }
    CHECK(errors == 0, "no call failed under 16 threads");
    bool s_ok = true, r_ok = true, p_ok = true, b_ok = true;
    for (size_t q = 0; q < nq; ++q) {
        s_ok &= same(got_search[q], want_search[q]);
        r_ok &= same(got_rerank[q], want_rerank[q]);
        p_ok &= same(got_probe[q], want_probe[q]);
        if (q % 16 == 0) b_ok &= same(got_brute[q], index.brute_force_search(queries.data() + q * dim, k));
    }
    CHECK(s_ok, "search from an OpenMP loop equals the batch call");
    CHECK(r_ok, "search_and_rerank from an OpenMP loop equals the batch call");
    CHECK(p_ok, "search_multiprobe from an OpenMP loop equals the batch call");
    CHECK(b_ok, "brute_force_search from an OpenMP loop equals the serial call");

    // searches keep running while another thread adds vectors (add excludes them while it works)
    const auto more = clustered(2000, dim, 40, 3);
    int errors2 = 0;
#pragma omp parallel sections reduction(+ : errors2)
    {
#pragma omp section
        {
            try { idx.add_batch(more.data(), 2000); } catch (const std::exception&) { ++errors2; }
        }
#pragma omp section
        {
            for (size_t q = 0; q < 64; ++q) {
                try {
                    auto r = index.search(queries.data() + q * dim, k, 100);
                    if (r.size() != k) ++errors2;
                } catch (const std::exception&) { ++errors2; }
            }
        }
    }
    CHECK(errors2 == 0 && idx.size() == n + 2000, "searches and add_batch from different threads");

    std::printf(failures ? "FAILED (%d)\n" : "ALL PASS\n", failures);
    return failures ? 1 : 0;
}
