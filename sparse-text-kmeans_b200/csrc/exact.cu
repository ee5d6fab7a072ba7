// Exact inner-product search and rerank over fp32 vectors: the reference's GPUBruteForce::search /
// ::rerank (src/cuda/gpu_encoder.cu:554-664, kernels :232-369) and the ground truth of its evaluation
// harness (evaluation/datasets/dataset_loader.hpp:187-212).  Results are the k smallest (-<q,x>, id),
// the dot product accumulated in fp32 in d order without fused multiply-add, so they equal a plain
// CPU loop bit for bit.  (The reference multiplies with cuBLAS and keeps a similarity matrix; here the
// top-k lists are kept in registers while the base vectors stream through shared memory once.)
#include <cmath>

#include "knn_common.cuh"

namespace cpb {
namespace {

using knn::kFull;

constexpr int kExQ = 8;        // queries per warp
constexpr int kExChunk = 32;   // dimensions per shared-memory stage
constexpr int kExMaxSplit = 64;

// float -> uint32 with the same order (and back)
__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// 16- or 4-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros and reads nothing
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool take) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(knn::smem_u32(dst)), "l"(src), "r"(take ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src, bool take) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(knn::smem_u32(dst)), "l"(src), "r"(take ? 4 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One warp owns kExQ queries, a lane owns CPL of the 32*CPL base vectors of a tile.  A stage of shared
// memory holds kExChunk dimensions of the tile's vectors and of the block's queries, rows kExRow floats
// apart (16-byte reads of a quarter warp fall into distinct banks); the next stage is copied in
// (cp.async) while the current one is multiplied.  gridDim.y splits the base vectors into contiguous
// ranges of whole tiles; with more than one range the lists go to part_key / part_id
// ([nq][gridDim.y][k]) and exact_merge_kernel finishes.
constexpr int kExWarps = 4;
constexpr int kExRow = kExChunk + 4;

template <int SLOTS, int CPL>
__global__ void __launch_bounds__(kExWarps * 32)
exact_topk_kernel(const float* __restrict__ base, uint64_t n, int dim, const float* __restrict__ queries, uint64_t nq,
                  uint32_t k, int aligned16, uint32_t* __restrict__ out_ids, float* __restrict__ out_dist,
                  uint32_t* __restrict__ part_key, uint32_t* __restrict__ part_id) {
    constexpr int TILE = 32 * CPL;
    constexpr int ROWS = TILE + kExWarps * kExQ;  // base rows, then query rows
    extern __shared__ __align__(16) float ex_smem[];  // [2][ROWS][kExRow]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t q_first = uint64_t(blockIdx.x) * kExWarps * kExQ;
    const uint64_t tiles = (n + TILE - 1) / TILE;
    const uint64_t t_begin = tiles * blockIdx.y / gridDim.y, t_end = tiles * (blockIdx.y + 1) / gridDim.y;
    const int nch = (dim + kExChunk - 1) / kExChunk;
    const uint64_t total = (t_end - t_begin) * nch;

    // stage `ci` = dimensions [d0, d0 + kExChunk) of tile t_begin + ci / nch
    auto issue = [&](uint64_t ci) {
        float* st = ex_smem + size_t(ci & 1) * ROWS * kExRow;
        const uint64_t c_first = (t_begin + ci / nch) * TILE;
        const int d0 = int(ci % nch) * kExChunk;
        if (aligned16) {
            for (int i = threadIdx.x; i < ROWS * (kExChunk / 4); i += kExWarps * 32) {
                const int row = i / (kExChunk / 4), j = (i % (kExChunk / 4)) * 4;
                const bool is_q = row >= TILE;
                const uint64_t r = is_q ? q_first + (row - TILE) : c_first + row;
                const bool take = r < (is_q ? nq : n) && d0 + j < dim;
                const float* src = (is_q ? queries : base) + (take ? r * dim + d0 + j : 0);
                cp_async16(st + row * kExRow + j, src, take);
            }
        } else {
            for (int i = threadIdx.x; i < ROWS * kExChunk; i += kExWarps * 32) {
                const int row = i / kExChunk, j = i % kExChunk;
                const bool is_q = row >= TILE;
                const uint64_t r = is_q ? q_first + (row - TILE) : c_first + row;
                const bool take = r < (is_q ? nq : n) && d0 + j < dim;
                const float* src = (is_q ? queries : base) + (take ? r * dim + d0 + j : 0);
                cp_async4(st + row * kExRow + j, src, take);
            }
        }
        cp_async_commit();
    };

    uint32_t ld[kExQ][SLOTS], li[kExQ][SLOTS], tau[kExQ];
#pragma unroll
    for (int q = 0; q < kExQ; ++q) {
        tau[q] = kFull;
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) ld[q][s] = kFull, li[q][s] = kInvalidNode;
    }
    float acc[kExQ][CPL];

    if (total) issue(0);
    for (uint64_t ci = 0; ci < total; ++ci) {
        if (ci + 1 < total) {
            issue(ci + 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();  // stage ci has landed for every thread
        const int ch = int(ci % nch);
        if (ch == 0) {
#pragma unroll
            for (int q = 0; q < kExQ; ++q)
#pragma unroll
                for (int m = 0; m < CPL; ++m) acc[q][m] = 0.0f;
        }
        const float* st = ex_smem + size_t(ci & 1) * ROWS * kExRow;
        const float* myq = st + (TILE + warp * kExQ) * kExRow;
        // whole groups of four dimensions; the padding of the last group multiplies 0 by 0
        const int dc = min(kExChunk, ((dim - ch * kExChunk) + 3) & ~3);
        for (int j = 0; j < dc; j += 4) {
            float4 x[CPL];
#pragma unroll
            for (int m = 0; m < CPL; ++m) x[m] = *reinterpret_cast<const float4*>(st + (lane + 32 * m) * kExRow + j);
#pragma unroll
            for (int q = 0; q < kExQ; ++q) {
                const float4 qv = *reinterpret_cast<const float4*>(myq + q * kExRow + j);
#pragma unroll
                for (int m = 0; m < CPL; ++m) {
                    float a = acc[q][m];
                    a = __fadd_rn(a, __fmul_rn(qv.x, x[m].x));
                    a = __fadd_rn(a, __fmul_rn(qv.y, x[m].y));
                    a = __fadd_rn(a, __fmul_rn(qv.z, x[m].z));
                    a = __fadd_rn(a, __fmul_rn(qv.w, x[m].w));
                    acc[q][m] = a;
                }
            }
        }
        if (ch == nch - 1) {
            // the tile is complete; candidates in ascending id order: m outer, lanes inner
            const uint64_t c_first = (t_begin + ci / nch) * TILE;
#pragma unroll
            for (int m = 0; m < CPL; ++m) {
                const uint64_t c = c_first + 32 * m + lane;
#pragma unroll
                for (int q = 0; q < kExQ; ++q) {
                    // 0 - dot: the negated dot product with one zero (+0) only
                    const uint32_t key = c < n ? order_key(__fsub_rn(0.0f, acc[q][m])) : kFull;
                    uint32_t mask = __ballot_sync(kFull, key < tau[q]);
                    while (mask) {
                        const int src = __ffs(mask) - 1;
                        mask &= mask - 1;
                        const uint32_t dd = __shfl_sync(kFull, key, src);
                        if (dd >= tau[q]) continue;  // tightened by an earlier lane
                        knn::list_insert<SLOTS>(ld[q], li[q], dd, uint32_t(c_first + 32 * m + src), lane);
                        tau[q] = knn::list_threshold<SLOTS>(ld[q], k - 1);
                    }
                }
            }
        }
        __syncthreads();  // stage ci is consumed before the next iteration copies over it
    }

#pragma unroll
    for (int q = 0; q < kExQ; ++q) {
        const uint64_t row = q_first + uint64_t(warp) * kExQ + q;
        if (row >= nq) continue;
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const uint32_t rank = s * 32 + lane;
            if (rank >= k) continue;
            if (gridDim.y == 1) {
                out_ids[row * k + rank] = li[q][s];
                out_dist[row * k + rank] = li[q][s] == kInvalidNode ? INFINITY : key_value(ld[q][s]);
            } else {
                const uint64_t o = (row * gridDim.y + blockIdx.y) * k + rank;
                part_key[o] = ld[q][s];
                part_id[o] = li[q][s];
            }
        }
    }
}

// One warp per query: the S partial lists (ascending id ranges, each sorted) merged into the final one.
template <int SLOTS>
__global__ void exact_merge_kernel(const uint32_t* __restrict__ part_key, const uint32_t* __restrict__ part_id, uint64_t nq,
                                   int S, uint32_t k, uint32_t* __restrict__ out_ids, float* __restrict__ out_dist) {
    const int lane = threadIdx.x & 31;
    const uint64_t q = uint64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (q >= nq) return;
    uint32_t ld[SLOTS], li[SLOTS], tau = kFull;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) ld[s] = kFull, li[s] = kInvalidNode;
    for (int y = 0; y < S; ++y) {
        const uint64_t o = (q * S + y) * k;
        for (uint32_t r0 = 0; r0 < k; r0 += 32) {
            const uint32_t r = r0 + lane;
            const uint32_t key = r < k ? part_key[o + r] : kFull;
            const uint32_t id = r < k ? part_id[o + r] : kInvalidNode;
            uint32_t mask = __ballot_sync(kFull, id != kInvalidNode && key < tau);
            while (mask) {
                const int src = __ffs(mask) - 1;
                mask &= mask - 1;
                const uint32_t dd = __shfl_sync(kFull, key, src);
                const uint32_t ii = __shfl_sync(kFull, id, src);
                if (dd >= tau) continue;
                knn::list_insert<SLOTS>(ld, li, dd, ii, lane);
                tau = knn::list_threshold<SLOTS>(ld, k - 1);
            }
        }
    }
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const uint32_t rank = s * 32 + lane;
        if (rank >= k) continue;
        out_ids[q * k + rank] = li[s];
        out_dist[q * k + rank] = li[s] == kInvalidNode ? INFINITY : key_value(ld[s]);
    }
}

// Rerank: one warp per query, a lane per candidate; candidate ids come in any order (ids >= n and the
// "no node" id are skipped), so the list is kept by the full (distance, id) order.
template <int SLOTS>
__global__ void rerank_kernel(const float* __restrict__ base, uint64_t n, int dim, const float* __restrict__ queries,
                              uint64_t nq, const uint32_t* __restrict__ cand, uint32_t num_cand, uint32_t k,
                              uint32_t* __restrict__ out_ids, float* __restrict__ out_dist) {
    const int lane = threadIdx.x & 31;
    const uint64_t q = uint64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (q >= nq) return;
    const float* qv = queries + q * dim;
    uint32_t ld[SLOTS], li[SLOTS];
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) ld[s] = kFull, li[s] = kInvalidNode;
    const bool vec4 = (dim & 3) == 0 && ((reinterpret_cast<uintptr_t>(base) | reinterpret_cast<uintptr_t>(queries)) & 15) == 0;
    for (uint32_t c0 = 0; c0 < num_cand; c0 += 32) {
        const uint32_t id = c0 + lane < num_cand ? cand[q * num_cand + c0 + lane] : kInvalidNode;
        const bool valid = id != kInvalidNode && id < n;
        uint32_t key = kFull;
        if (valid) {
            const float* x = base + uint64_t(id) * dim;
            float dot = 0.0f;
            if (vec4) {
                for (int d = 0; d < dim; d += 4) {
                    const float4 a = __ldg(reinterpret_cast<const float4*>(qv + d));
                    const float4 b = __ldg(reinterpret_cast<const float4*>(x + d));
                    dot = __fadd_rn(dot, __fmul_rn(a.x, b.x));
                    dot = __fadd_rn(dot, __fmul_rn(a.y, b.y));
                    dot = __fadd_rn(dot, __fmul_rn(a.z, b.z));
                    dot = __fadd_rn(dot, __fmul_rn(a.w, b.w));
                }
            } else {
                for (int d = 0; d < dim; ++d) dot = __fadd_rn(dot, __fmul_rn(__ldg(qv + d), __ldg(x + d)));
            }
            key = order_key(__fsub_rn(0.0f, dot));
        }
        uint32_t mask = __ballot_sync(kFull, valid);
        while (mask) {
            const int src = __ffs(mask) - 1;
            mask &= mask - 1;
            const uint32_t dd = __shfl_sync(kFull, key, src);
            const uint32_t ii = __shfl_sync(kFull, id, src);
            const int p = knn::list_rank_keyed<SLOTS>(ld, li, dd, ii);
            if (p < int(k)) knn::list_place<SLOTS>(ld, li, p, dd, ii, lane);
        }
    }
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const uint32_t rank = s * 32 + lane;
        if (rank >= k) continue;
        out_ids[q * k + rank] = li[s];
        out_dist[q * k + rank] = li[s] == kInvalidNode ? INFINITY : key_value(ld[s]);
    }
}

template <int SLOTS, int CPL>
int launch_exact_t(cphnsw_b200_index* h, const float* d_base, uint64_t n, const float* d_q, uint64_t nq, uint32_t k,
                   uint32_t* d_ids, float* d_dist, cudaStream_t st) {
    constexpr int TILE = 32 * CPL;
    const int dim = int(h->dim);
    const size_t smem = size_t(2) * (TILE + kExWarps * kExQ) * kExRow * sizeof(float);
    const uint64_t blocks = (nq + uint64_t(kExWarps) * kExQ - 1) / (uint64_t(kExWarps) * kExQ);
    const uint64_t tiles = (n + TILE - 1) / TILE;
    // enough blocks for four waves of four blocks per SM (a short tail); every range holds at least four tiles
    uint64_t S = (4 * uint64_t(h->sm_count) * 4 + blocks - 1) / blocks;
    if (S > tiles / 4) S = tiles / 4;
    if (S > kExMaxSplit) S = kExMaxSplit;
    if (S < 1) S = 1;
    uint32_t *pk = nullptr, *pi = nullptr;
    if (S > 1) {
        CPB_TRY(h->s_pad.reserve(nq * S * k * 4 + 16));
        CPB_TRY(h->s_pad2.reserve(nq * S * k * 4 + 16));
        pk = h->s_pad.as<uint32_t>(), pi = h->s_pad2.as<uint32_t>();
    }
    const int aligned16 =
        (dim & 3) == 0 && ((reinterpret_cast<uintptr_t>(d_base) | reinterpret_cast<uintptr_t>(d_q)) & 15) == 0 ? 1 : 0;
    CPB_CUDA(cudaFuncSetAttribute(exact_topk_kernel<SLOTS, CPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    exact_topk_kernel<SLOTS, CPL><<<dim3(unsigned(blocks), unsigned(S)), kExWarps * 32, smem, st>>>(
        d_base, n, dim, d_q, nq, k, aligned16, d_ids, d_dist, pk, pi);
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    if (S > 1) {
        exact_merge_kernel<SLOTS><<<unsigned((nq + 3) / 4), 128, 0, st>>>(pk, pi, nq, int(S), k, d_ids, d_dist);
        h->launches++;
        CPB_CUDA(cudaGetLastError());
    }
    return 0;
}

}  // namespace

// ids uint32[nq][k], dist float[nq][k] (device): the k smallest (-<q,x>, id) over base[n][dim]; rows are
// padded with (no node, +inf) when n < k
int launch_exact_search(cphnsw_b200_index* h, const float* d_base, uint64_t n, const float* d_q, uint64_t nq, uint32_t k,
                        uint32_t* d_ids, float* d_dist, cudaStream_t st) {
    if (nq == 0) return 0;
    if (k == 0 || k > 128) {
        set_error("exact_search: k must be in 1..128 (got %u)", k);
        return CPHNSW_B200_E_INVALID;
    }
    if (nq > 0x7fffffffull * 8) {
        set_error("exact_search: too many queries");
        return CPHNSW_B200_E_INVALID;
    }
    if (k <= 32) return launch_exact_t<1, 4>(h, d_base, n, d_q, nq, k, d_ids, d_dist, st);
    if (k <= 64) return launch_exact_t<2, 4>(h, d_base, n, d_q, nq, k, d_ids, d_dist, st);
    return launch_exact_t<4, 2>(h, d_base, n, d_q, nq, k, d_ids, d_dist, st);
}

// ids / dist as above from the candidates cand[nq][num_cand] (device)
int launch_rerank(cphnsw_b200_index* h, const float* d_base, uint64_t n, const float* d_q, uint64_t nq, const uint32_t* d_cand,
                  uint32_t num_cand, uint32_t k, uint32_t* d_ids, float* d_dist, cudaStream_t st) {
    if (nq == 0) return 0;
    if (k == 0 || k > 128) {
        set_error("rerank: k must be in 1..128 (got %u)", k);
        return CPHNSW_B200_E_INVALID;
    }
    const unsigned grid = unsigned((nq + 3) / 4);
    const int dim = int(h->dim);
    if (k <= 32) rerank_kernel<1><<<grid, 128, 0, st>>>(d_base, n, dim, d_q, nq, d_cand, num_cand, k, d_ids, d_dist);
    else if (k <= 64) rerank_kernel<2><<<grid, 128, 0, st>>>(d_base, n, dim, d_q, nq, d_cand, num_cand, k, d_ids, d_dist);
    else rerank_kernel<4><<<grid, 128, 0, st>>>(d_base, n, dim, d_q, nq, d_cand, num_cand, k, d_ids, d_dist);
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace cpb
