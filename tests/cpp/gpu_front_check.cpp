// Checks of the C++ fronts that mirror the reference's GPU classes (GPUEncoder, GPUBruteForce,
// GPUKNNGraphBuilder, KNNEdgeList), modelled on the reference's own debug programs
// (evaluation/debug_gpu_knn.cpp:42-68: no self loops, ids in range; evaluation/debug_code_storage.cpp:63-105:
// stored code == fresh code).  Needs a B200.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

#include "cphnsw/cuda/gpu_knn_graph.cuh"
#include "cphnsw/index/cp_hnsw_index.hpp"

using namespace cphnsw;

static int failures = 0;
#define CHECK(cond, what)                                             \
    do {                                                              \
        if (cond) std::printf("[PASS] %s\n", what);                   \
        else { std::printf("[FAIL] %s\n", what); ++failures; }        \
    } while (0)

static std::vector<float> unit_vectors(size_t n, size_t dim, uint64_t seed) {
    std::mt19937_64 rng(seed);
    std::normal_distribution<float> g(0.f, 1.f);
    std::vector<float> v(n * dim);
    for (size_t i = 0; i < n; ++i) {
        float s = 0;
        for (size_t d = 0; d < dim; ++d) { v[i * dim + d] = g(rng); s += v[i * dim + d] * v[i * dim + d]; }
        const float inv = 1.0f / std::sqrt(s);
        for (size_t d = 0; d < dim; ++d) v[i * dim + d] *= inv;
    }
    return v;
}

int main() {
    const size_t dim = 100, n = 3000, nq = 40;
    auto base = unit_vectors(n, dim, 1), queries = unit_vectors(nq, dim, 2);

    // ---- GPUEncoder ----
    cuda::GPUEncoder<uint8_t, 32> enc(dim);
    CHECK(enc.dim() == dim && enc.padded_dim() == 128, "GPUEncoder dim / padded_dim");
    std::vector<uint8_t> codes(n * 32), qcodes(nq * 32), qcodes2(nq * 32);
    enc.encode_batch(base.data(), n, codes.data());
    {
        CPHNSWIndex<uint8_t, 32> index(dim, 16, 200);
        index.add_batch_parallel(base.data(), n);
        bool same = true;
        for (size_t i = 0; i < n && same; i += 97) {
            auto c = index.get_code(NodeId(i));
            for (size_t r = 0; r < 32; ++r) same &= c.components[r] == codes[i * 32 + r];
        }
        CHECK(same, "GPUEncoder::encode_batch equals the codes the index stores");
    }
    std::vector<float> mags(nq * 32);
    enc.encode_queries_batch(queries.data(), nq, qcodes.data(), mags.data());
    enc.encode_batch(queries.data(), nq, qcodes2.data());
    CHECK(qcodes == qcodes2, "encode_queries_batch codes equal encode_batch codes");
    CHECK(std::all_of(mags.begin(), mags.end(), [](float m) { return m > 0.f && std::isfinite(m); }), "query magnitudes are positive");
    {
        // device form: vectors zero padded to padded_dim
        std::vector<float> padded(n * 128, 0.f);
        for (size_t i = 0; i < n; ++i) std::copy(base.begin() + i * dim, base.begin() + (i + 1) * dim, padded.begin() + i * 128);
        float* d_x = nullptr;
        uint8_t* d_c = nullptr;
        cudaMalloc(reinterpret_cast<void**>(&d_x), padded.size() * 4);
        cudaMalloc(reinterpret_cast<void**>(&d_c), codes.size());
        cudaMemcpy(d_x, padded.data(), padded.size() * 4, cudaMemcpyHostToDevice);
        enc.encode_batch_device(d_x, n, d_c);
        std::vector<uint8_t> back(codes.size());
        cudaMemcpy(back.data(), d_c, back.size(), cudaMemcpyDeviceToHost);
        CHECK(back == codes, "encode_batch_device on padded vectors equals encode_batch");
        cuda::GPUEncoder<uint8_t, 32> moved(std::move(enc));
        moved.encode_batch(queries.data(), nq, qcodes2.data());
        CHECK(qcodes == qcodes2, "a moved GPUEncoder encodes the same");
        cudaFree(d_x);
        cudaFree(d_c);
    }

    // ---- GPUBruteForce ----
    const size_t k = 10;
    cuda::GPUBruteForce bf(dim, n);
    bf.set_base_vectors(base.data(), n);
    std::vector<uint32_t> ids(nq * k);
    std::vector<float> dist(nq * k);
    bf.search(queries.data(), nq, k, ids.data(), dist.data());
    {
        bool same = true;
        for (size_t q = 0; q < nq && same; ++q) {
            std::vector<std::pair<float, uint32_t>> all(n);
            for (size_t i = 0; i < n; ++i) {
                float dot = 0.f;
                for (size_t d = 0; d < dim; ++d) dot += queries[q * dim + d] * base[i * dim + d];
                all[i] = {-dot, uint32_t(i)};
            }
            std::sort(all.begin(), all.end());
            for (size_t t = 0; t < k; ++t) same &= ids[q * k + t] == all[t].second && dist[q * k + t] == all[t].first;
        }
        CHECK(same, "GPUBruteForce::search equals a CPU loop (ids and distances)");
    }
    {
        // every id as a candidate, in reverse order: rerank must find the same top-k
        std::vector<uint32_t> cand(nq * n);
        for (size_t q = 0; q < nq; ++q)
            for (size_t i = 0; i < n; ++i) cand[q * n + i] = uint32_t(n - 1 - i);
        std::vector<uint32_t> ids2(nq * k);
        std::vector<float> dist2(nq * k);
        bf.rerank(queries.data(), cand.data(), nq, n, k, ids2.data(), dist2.data());
        CHECK(ids2 == ids && dist2 == dist, "GPUBruteForce::rerank over all ids equals search");
    }

    // ---- GPUKNNGraphBuilder / KNNEdgeList ----
    const size_t kk = 32;
    cuda::GPUKNNGraphBuilder knn(dim, kk);
    std::vector<uint32_t> nbrs(n * kk), nbrs2(n * kk);
    std::vector<float> nd(n * kk);
    knn.build(base.data(), n, nbrs.data(), nd.data());
    {
        bool ok = true;
        for (size_t i = 0; i < n; ++i)
            for (size_t j = 0; j < kk; ++j) {
                ok &= nbrs[i * kk + j] != i && nbrs[i * kk + j] < n;
                if (j) ok &= nd[i * kk + j - 1] <= nd[i * kk + j];
            }
        CHECK(ok, "kNN graph: no self loops, ids in range, distances ascending");
        // distances are code distances
        size_t i = 17, j = 5, diff = 0;
        for (size_t r = 0; r < 32; ++r) diff += codes[i * 32 + r] != codes[size_t(nbrs[i * kk + j]) * 32 + r];
        CHECK(nd[i * kk + j] == float(diff), "kNN distances are the numbers of differing code components");
    }
    {
        float* d_x = nullptr;
        cudaMalloc(reinterpret_cast<void**>(&d_x), base.size() * 4);
        cudaMemcpy(d_x, base.data(), base.size() * 4, cudaMemcpyHostToDevice);
        knn.build_device(d_x, n, nbrs2.data());
        cudaFree(d_x);
        CHECK(nbrs2 == nbrs, "build_device equals build");
    }
    {
        auto e = cuda::KNNEdgeList::from_matrix(nbrs.data(), nd.data(), n, kk);
        auto r = e.get_neighbors(123);
        bool ok = e.num_nodes == n && e.k == kk && e.sources.size() == n * kk && r.second == kk;
        for (size_t j = 0; j < kk && ok; ++j) ok = r.first[j] == nbrs[123 * kk + j];
        CHECK(ok, "KNNEdgeList::from_matrix / get_neighbors");
        // a tiny graph: rows are padded when N - 1 < k, the edge list drops the padding
        cuda::GPUKNNGraphBuilder small(dim, 8);
        std::vector<uint32_t> sn(5 * 8);
        small.build(base.data(), 5, sn.data());
        auto se = cuda::KNNEdgeList::from_matrix(sn.data(), nullptr, 5, 8);
        CHECK(sn[4] == CPHNSW_B200_INVALID_NODE && se.targets.size() == 20 && se.get_neighbors(2).second == 4,
              "rows padded with 0xFFFFFFFF when N - 1 < k");
    }
    std::printf("%s (%d failures)\n", failures ? "FAILED" : "ALL PASS", failures);
    return failures ? 1 : 0;
}
