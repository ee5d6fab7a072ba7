// Diagnostics of the legacy index that its evaluation programs call around the hot path:
// verify_connectivity (evaluation/eval_main.cpp:52), calibrate / search_calibrated
// (evaluation/eval_main.cpp:128-189) and the scoring half of brute_force_search
// (evaluation/eval_sift.cpp:283; the scan itself is the search kernel in scan-only mode).
// The legacy sources are absent from the reference tree; the behaviour follows the call sites.
#include "search_common.cuh"

namespace cpb {
namespace {

using namespace srch;

// ---- connectivity: level-synchronous breadth-first search over the directed adjacency ---------------
__global__ void bfs_seed_kernel(const uint32_t* __restrict__ entry, uint32_t n_entry, uint64_t n, uint8_t* __restrict__ seen,
                                uint32_t* __restrict__ frontier, uint32_t* __restrict__ counters) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_entry) return;
    const uint32_t v = entry[i];
    if (v >= n) return;
    // one byte per node inside a 32-bit word: the first thread to set the byte owns the node
    uint32_t* word = reinterpret_cast<uint32_t*>(seen + (v & ~3u));
    const uint32_t bit = 1u << (8 * (v & 3u));
    if (atomicOr(word, bit) & bit) return;
    frontier[atomicAdd(counters, 1u)] = v;
}

__global__ void bfs_level_kernel(const uint32_t* __restrict__ adj, uint64_t n, int M, uint8_t* __restrict__ seen,
                                 const uint32_t* __restrict__ frontier, uint32_t n_frontier,
                                 uint32_t* __restrict__ next, uint32_t* __restrict__ next_count) {
    const uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= uint64_t(n_frontier) * M) return;
    const uint32_t v = frontier[t / M];
    const uint32_t w = adj[uint64_t(v) * M + t % M];
    if (w >= n) return;
    uint32_t* word = reinterpret_cast<uint32_t*>(seen + (w & ~3u));
    const uint32_t bit = 1u << (8 * (w & 3u));
    if (atomicOr(word, bit) & bit) return;
    next[atomicAdd(next_count, 1u)] = w;
}

// ---- calibration samples: one thread per pair (u, v) ------------------------------------------------
// x = asymmetric CP score of v's code against the rotated vectors of u (the add tree of the search
// kernels), y = -<x_u, x_v> accumulated in d order in fp32.
template <bool U16>
__global__ void calibration_samples_kernel(const float* __restrict__ tables, int K, int P, const void* __restrict__ codes,
                                           const float* __restrict__ vectors, int dim, const uint32_t* __restrict__ u,
                                           const uint32_t* __restrict__ v, uint32_t m, float* __restrict__ x,
                                           float* __restrict__ y) {
    const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= m) return;
    x[s] = asym_distance_lane<U16>(tables + size_t(s) * K * P, codes, v[s], K, P);
    const float* a = vectors + size_t(u[s]) * dim;
    const float* b = vectors + size_t(v[s]) * dim;
    float dot = 0.0f;
    for (int d = 0; d < dim; ++d) dot = __fadd_rn(dot, __fmul_rn(a[d], b[d]));
    y[s] = -dot;
}

// ---- calibrated distances: d -> alpha * d + beta (estimate of the true distance), +inf kept ---------
__global__ void affine_kernel(float* __restrict__ d, uint64_t n, float alpha, float beta) {
    const uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = d[i];
    if (v != INFINITY) d[i] = __fadd_rn(__fmul_rn(alpha, v), beta);
}

// ---- packed sign bits: one thread per (node, 64-bit word); bit r = bit 0 of component r ---------------
__global__ void pack_sign_bits_kernel(const unsigned char* __restrict__ codes, uint64_t n, int K, int comp_bytes,
                                      unsigned long long* __restrict__ out) {
    const int nw = (K + 63) / 64;
    const uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= n * nw) return;
    const uint64_t node = t / nw;
    const int w = int(t % nw);
    const unsigned char* row = codes + node * uint64_t(K) * comp_bytes;
    unsigned long long bits = 0;
    for (int b = 0; b < 64 && w * 64 + b < K; ++b)
        if (row[size_t(w * 64 + b) * comp_bytes] & 1u) bits |= 1ull << b;  // the low byte of a component holds the sign
    out[t] = bits;
}

}  // namespace

int launch_pack_sign_bits(cphnsw_b200_index* h, const void* d_codes, uint64_t n, uint64_t* d_out, cudaStream_t st) {
    const uint64_t threads = n * ((h->K + 63) / 64);
    if (threads == 0) return 0;
    pack_sign_bits_kernel<<<unsigned((threads + 255) / 256), 256, 0, st>>>(static_cast<const unsigned char*>(d_codes), n, int(h->K),
                                                                          int(h->comp_bytes),
                                                                          reinterpret_cast<unsigned long long*>(d_out));
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

// Number of nodes reachable from the entry nodes (the entry nodes included).
int launch_connectivity(cphnsw_b200_index* h, uint64_t* reachable, cudaStream_t st) {
    const uint64_t n = h->n;
    const int M = int(h->M);
    const size_t seen_bytes = (size_t(n) + 3) & ~size_t(3);
    CPB_TRY(h->s_pad.reserve(seen_bytes + 16));
    CPB_TRY(h->s_in.reserve(size_t(n) * 4 + 16));
    CPB_TRY(h->s_in2.reserve(size_t(n) * 4 + 16));
    uint8_t* seen = h->s_pad.as<uint8_t>();
    uint32_t* front[2] = {h->s_in.as<uint32_t>(), h->s_in2.as<uint32_t>()};
    uint32_t* counters = h->d_status.as<uint32_t>() + 4;  // two words: sizes of the two frontiers
    CPB_CUDA(cudaMemsetAsync(seen, 0, seen_bytes, st));
    CPB_CUDA(cudaMemsetAsync(counters, 0, 8, st));
    if (h->n_entry) {
        bfs_seed_kernel<<<(h->n_entry + 255) / 256, 256, 0, st>>>(h->d_entry.as<uint32_t>(), h->n_entry, n, seen, front[0], counters);
        h->launches++;
        CPB_CUDA(cudaGetLastError());
    }
    uint64_t total = 0;
    int cur = 0;
    for (uint64_t level = 0; level <= n; ++level) {  // at most n levels: each adds at least one node
        uint32_t nf = 0;
        CPB_CUDA(cudaMemcpyAsync(&nf, counters + cur, 4, cudaMemcpyDeviceToHost, st));
        CPB_CUDA(cudaStreamSynchronize(st));
        if (nf == 0) break;
        total += nf;
        CPB_CUDA(cudaMemsetAsync(counters + (cur ^ 1), 0, 4, st));
        const uint64_t threads = uint64_t(nf) * M;
        bfs_level_kernel<<<unsigned((threads + 255) / 256), 256, 0, st>>>(h->d_adj.as<uint32_t>(), n, M, seen, front[cur], nf,
                                                                        front[cur ^ 1], counters + (cur ^ 1));
        h->launches++;
        CPB_CUDA(cudaGetLastError());
        cur ^= 1;
    }
    *reachable = total;
    return 0;
}

// x[m], y[m] (device) for the pairs u[m], v[m] (device); tables = rotated vectors of the u nodes
int launch_calibration_samples(cphnsw_b200_index* h, const float* d_tables, const uint32_t* d_u, const uint32_t* d_v,
                               uint32_t m, float* d_x, float* d_y, cudaStream_t st) {
    if (m == 0) return 0;
    const unsigned grid = (m + 127) / 128;
    if (h->comp_bytes == 2)
        calibration_samples_kernel<true><<<grid, 128, 0, st>>>(d_tables, int(h->K), int(h->P), h->d_codes.p, h->d_vectors.as<float>(),
                                                              int(h->dim), d_u, d_v, m, d_x, d_y);
    else
        calibration_samples_kernel<false><<<grid, 128, 0, st>>>(d_tables, int(h->K), int(h->P), h->d_codes.p, h->d_vectors.as<float>(),
                                                               int(h->dim), d_u, d_v, m, d_x, d_y);
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

int launch_affine(cphnsw_b200_index* h, float* d_dist, uint64_t n, float alpha, float beta, cudaStream_t st) {
    if (n == 0) return 0;
    affine_kernel<<<unsigned((n + 255) / 256), 256, 0, st>>>(d_dist, n, alpha, beta);
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace cpb
