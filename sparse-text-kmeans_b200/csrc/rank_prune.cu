// Rank-based pruning of a kNN graph (the CAGRA graph optimisation the legacy index ran behind
// build_with_gpu_knn(..., prune = true, alpha); parameter include/cphnsw/core/types.hpp:399-400,
// use evaluation/test_gpu_build.cpp:168-174; the legacy source is absent, the rule is the paper's,
// resources/arXiv-2308.15136v2/consolidated.tex:298-340).  No distance is computed: only the
// positions ("ranks", 1 = nearest) of nodes in the distance-ordered kNN lists are used.
//
//   1. reorder:  for node X with list L_X, a two-hop route X -> Z -> Y (Z, Y in L_X, Y in L_Z) is a
//      detour of the edge X -> Y when  alpha * max(rank_X(Z), rank_Z(Y)) < rank_X(Y)
//      (alpha = 1 is the paper's condition; the legacy "detour threshold" alpha >= 1 asks for a
//      margin).  The edges of X are ordered by (number of detours, initial rank) and the first M kept.
//   2. reverse:  node P receives every X that kept P, ordered by (rank of P in X's kept list, X).
//   3. merge:    the kept list and the reverse list of P are interleaved, kept list first, an id
//      taken once, until M links are chosen; when one list runs out the other goes on alone.
#include "common.cuh"

namespace cpb {
namespace {

constexpr uint32_t kFull = 0xffffffffu;
constexpr int kRpWarps = 4;
constexpr int kRpMaxK = 64;

// One warp per node X of [row_begin, row_end): detour counts of its k candidates, then the M
// first by (count, initial rank) -> out[X - row_begin][M].
__global__ void __launch_bounds__(kRpWarps * 32)
rank_reorder_kernel(const uint32_t* __restrict__ cand, uint64_t n, uint32_t k, uint64_t row_begin, uint64_t row_end,
                    uint32_t M, float alpha, uint32_t* __restrict__ out) {
    __shared__ uint32_t lx[kRpWarps][kRpMaxK];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t X = row_begin + uint64_t(blockIdx.x) * kRpWarps + warp;
    if (X >= row_end) return;
    const uint32_t* row = cand + X * k;
    uint32_t yj[2], cnt[2] = {0u, 0u};
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        const uint32_t j = uint32_t(lane + 32 * s);
        uint32_t y = j < k ? row[j] : kInvalidNode;
        if (y >= n) y = kInvalidNode;
        yj[s] = y;
        lx[warp][j] = y;
    }
    __syncwarp();
    for (uint32_t i = 0; i < k; ++i) {
        const uint32_t Z = lx[warp][i];
        if (Z == kInvalidNode) continue;
        const uint32_t* zrow = cand + uint64_t(Z) * k;
        uint32_t z[2];
        z[0] = uint32_t(lane) < k ? __ldg(zrow + lane) : kInvalidNode;
        z[1] = uint32_t(lane) + 32 < k ? __ldg(zrow + lane + 32) : kInvalidNode;
        for (uint32_t p = 0; p < k; ++p) {
            const uint32_t y = __shfl_sync(kFull, p < 32 ? z[0] : z[1], int(p & 31));
            if (y >= n) continue;
            const float thr = alpha * float(max(i, p) + 1);  // ranks count from 1
#pragma unroll
            for (int s = 0; s < 2; ++s)
                if (yj[s] == y && thr < float(lane + 32 * s + 1)) ++cnt[s];
        }
    }
    // position of every candidate in the order (count, initial rank); absent candidates go last
    uint32_t key[2], pos[2] = {0u, 0u};
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        const uint32_t c = yj[s] == kInvalidNode ? 0xFFFFFFu : cnt[s];
        key[s] = (c << 6) | uint32_t(lane + 32 * s);
    }
    for (int t = 0; t < 64; ++t) {
        const uint32_t other = __shfl_sync(kFull, t < 32 ? key[0] : key[1], t & 31);
        pos[0] += other < key[0];
        pos[1] += other < key[1];
    }
    uint32_t* o = out + (X - row_begin) * uint64_t(M);
#pragma unroll
    for (int s = 0; s < 2; ++s)
        if (pos[s] < M) o[pos[s]] = yj[s];
}

// reverse lists of the nodes of [row_begin, row_end): in-degree, segments, entries
__global__ void rank_rev_count_kernel(const uint32_t* __restrict__ kept, uint64_t edges, uint64_t row_begin,
                                      uint64_t row_end, uint32_t* __restrict__ cnt) {
    const uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= edges) return;
    const uint32_t v = kept[t];
    if (v >= row_begin && v < row_end) atomicAdd(cnt + (v - row_begin), 1u);
}
__global__ void rank_rev_alloc_kernel(const uint32_t* __restrict__ cnt, uint64_t rows, uint32_t* __restrict__ seg,
                                      unsigned long long* __restrict__ used) {
    const uint64_t v = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (v >= rows) return;
    // the place of a segment depends on the order of the atomics; what is read from it does not
    seg[v] = cnt[v] ? uint32_t(atomicAdd(used, (unsigned long long)cnt[v])) : 0u;
}
__global__ void rank_rev_fill_kernel(const uint32_t* __restrict__ kept, uint64_t edges, uint32_t M, uint64_t row_begin,
                                     uint64_t row_end, const uint32_t* __restrict__ seg, uint32_t* __restrict__ fill,
                                     uint64_t* __restrict__ inc) {
    const uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= edges) return;
    const uint32_t v = kept[t];
    if (v < row_begin || v >= row_end) return;
    const uint64_t X = t / M, r = t % M;
    inc[seg[v - row_begin] + atomicAdd(fill + (v - row_begin), 1u)] = (r << 32) | X;
}

// One warp per node P: the M smallest reverse entries by (rank, X), then the interleaving merge.
__global__ void __launch_bounds__(kRpWarps * 32)
rank_merge_kernel(const uint32_t* __restrict__ kept, uint64_t n, uint32_t M, uint64_t row_begin, uint64_t row_end,
                  const uint32_t* __restrict__ cnt, const uint32_t* __restrict__ seg, const uint64_t* __restrict__ inc,
                  uint32_t* __restrict__ adj) {
    __shared__ uint32_t la[kRpWarps][64], lb[kRpWarps][64], lo[kRpWarps][64];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t P = row_begin + uint64_t(blockIdx.x) * kRpWarps + warp;
    if (P >= row_end) return;
    const uint64_t none = ~0ull;
    // sorted list of the 64 smallest keys across the warp: rank 32 * s + lane in kk[s]
    uint64_t kk[2] = {none, none};
    const uint32_t total = cnt[P - row_begin];
    const uint64_t* mine = inc + seg[P - row_begin];
    for (uint32_t c0 = 0; c0 < total; c0 += 32) {
        const uint32_t c = c0 + lane;
        const uint64_t key = c < total ? mine[c] : none;
        uint32_t live = __ballot_sync(kFull, key != none);
        while (live) {
            const int src = __ffs(live) - 1;
            live &= live - 1;
            const uint64_t k1 = __shfl_sync(kFull, key, src);
            int p = 0;
#pragma unroll
            for (int s = 0; s < 2; ++s) p += __popc(__ballot_sync(kFull, kk[s] < k1));
            if (p >= 64) continue;
#pragma unroll
            for (int s = 1; s >= 0; --s) {
                uint64_t up = __shfl_up_sync(kFull, kk[s], 1);
                if (s > 0) {
                    const uint64_t carry = __shfl_sync(kFull, kk[s - 1], 31);
                    if (lane == 0) up = carry;
                }
                const int rank = s * 32 + lane;
                if (rank > p) kk[s] = up;
                else if (rank == p) kk[s] = k1;
            }
        }
    }
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        const uint32_t j = uint32_t(lane + 32 * s);
        uint32_t a = j < M ? kept[P * M + j] : kInvalidNode;
        if (a >= n) a = kInvalidNode;
        la[warp][j] = a;
        lb[warp][j] = (kk[s] == none || j >= M) ? kInvalidNode : uint32_t(kk[s]);
        lo[warp][j] = kInvalidNode;
    }
    __syncwarp();
    // every lane runs the same merge; lane 0 writes
    uint32_t ia = 0, ib = 0, no = 0;
    auto taken = [&](uint32_t id) {
        return __any_sync(kFull, lo[warp][lane] == id || lo[warp][lane + 32] == id);
    };
    int turn = 0;
    while (no < M) {
        while (ia < 64 && (la[warp][ia] == kInvalidNode || taken(la[warp][ia]))) {
            if (la[warp][ia] == kInvalidNode) { ia = 64; break; }
            ++ia;
        }
        while (ib < 64 && (lb[warp][ib] == kInvalidNode || taken(lb[warp][ib]))) {
            if (lb[warp][ib] == kInvalidNode) { ib = 64; break; }
            ++ib;
        }
        if (ia >= 64 && ib >= 64) break;
        const bool from_a = ib >= 64 || (ia < 64 && turn == 0);
        const uint32_t id = from_a ? la[warp][ia] : lb[warp][ib];
        if (from_a) ++ia; else ++ib;
        __syncwarp();
        if (lane == 0) lo[warp][no] = id;
        __syncwarp();
        ++no;
        turn ^= 1;
    }
    uint32_t* o = adj + (P - row_begin) * uint64_t(M);
    for (uint32_t j = lane; j < M; j += 32) o[j] = lo[warp][j];
}

}  // namespace

int launch_rank_reorder(cphnsw_b200_index* h, uint64_t n, const uint32_t* d_cand, uint32_t k, uint64_t row_begin,
                        uint64_t row_end, uint32_t M, float alpha, uint32_t* d_kept, cudaStream_t st) {
    if (row_end <= row_begin) return 0;
    if (k == 0 || k > kRpMaxK || M == 0 || M > 64 || row_end > n) {
        set_error("rank pruning: need 1 <= k <= 64, 1 <= M <= 64 and rows within n (got k=%u M=%u)", k, M);
        return CPHNSW_B200_E_INVALID;
    }
    const uint64_t rows = row_end - row_begin;
    LaunchTimer timer(h, kKernelSelect, st);
    rank_reorder_kernel<<<unsigned((rows + kRpWarps - 1) / kRpWarps), kRpWarps * 32, 0, st>>>(d_cand, n, k, row_begin, row_end,
                                                                                           M, alpha, d_kept);
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

int launch_rank_merge(cphnsw_b200_index* h, uint64_t n, const uint32_t* d_kept, uint32_t M, uint64_t row_begin,
                      uint64_t row_end, uint32_t* d_adj, cudaStream_t st) {
    if (row_end <= row_begin) return 0;
    if (M == 0 || M > 64 || row_end > n) {
        set_error("rank pruning: need 1 <= M <= 64 and rows within n");
        return CPHNSW_B200_E_INVALID;
    }
    const uint64_t rows = row_end - row_begin, edges = n * M;
    // scratch: cnt, seg, fill [rows] (uint32), used (uint64), inc [<= edges] (uint64)
    const size_t head = (size_t(rows) * 3 * 4 + 8 + 15) / 16 * 16;
    CPB_TRY(h->s_rank.reserve(head + size_t(edges) * 8 + 16));
    uint32_t* cnt = h->s_rank.as<uint32_t>();
    uint32_t* seg = cnt + rows;
    uint32_t* fill = seg + rows;
    unsigned long long* used = reinterpret_cast<unsigned long long*>(h->s_rank.as<unsigned char>() + head - 8);
    uint64_t* inc = reinterpret_cast<uint64_t*>(h->s_rank.as<unsigned char>() + head);
    CPB_CUDA(cudaMemsetAsync(cnt, 0, head, st));
    const unsigned eb = unsigned((edges + 255) / 256);
    rank_rev_count_kernel<<<eb, 256, 0, st>>>(d_kept, edges, row_begin, row_end, cnt);
    rank_rev_alloc_kernel<<<unsigned((rows + 255) / 256), 256, 0, st>>>(cnt, rows, seg, used);
    rank_rev_fill_kernel<<<eb, 256, 0, st>>>(d_kept, edges, M, row_begin, row_end, seg, fill, inc);
    LaunchTimer timer(h, kKernelSelect, st);
    rank_merge_kernel<<<unsigned((rows + kRpWarps - 1) / kRpWarps), kRpWarps * 32, 0, st>>>(d_kept, n, M, row_begin, row_end, cnt,
                                                                                         seg, inc, d_adj);
    h->launches += 4;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

// all rows on one device: reorder everything, then reverse + merge
int launch_rank_prune(cphnsw_b200_index* h, uint64_t n, const uint32_t* d_cand, uint32_t k, uint32_t M, float alpha,
                      uint32_t* d_adj, cudaStream_t st) {
    CPB_TRY(h->s_kept.reserve(size_t(n) * M * 4 + 16));
    CPB_TRY(launch_rank_reorder(h, n, d_cand, k, 0, n, M, alpha, h->s_kept.as<uint32_t>(), st));
    return launch_rank_merge(h, n, h->s_kept.as<uint32_t>(), M, 0, n, d_adj, st);
}

}  // namespace cpb
