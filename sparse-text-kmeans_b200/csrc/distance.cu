// CP-code distance, brute-force code-distance kNN graph and select_neighbors pruning.
//
// Distance between two codes = number of the K components that differ (the legacy
// hamming_distance(CPCode,CPCode); use sites evaluation/debug_estimator.cpp:149,172).  All three
// kernels work on code rows padded to 4, 8 or 16 32-bit words (zero padding on both sides never
// differs) and count differing bytes / halfwords branch-free in SWAR form: a per-lane "nonzero"
// flag is raised in the top bit of each byte of (a XOR b), flags of up to 8 (16) words are
// packed into one register by shifting, and one popcount finishes the row.
//
// kNN graph (replaces GPUKNNGraphBuilder::build, src/cuda/gpu_knn_graph.cu:330-415, with the
// CP-code metric): each warp owns Q query rows and sweeps every candidate; candidate tiles are
// brought into shared memory by bulk asynchronous copies (cp.async.bulk + mbarrier, two stages)
// issued by one thread; the running k+1 best of each row live in registers, spread over the
// warp in sorted order, and are updated by shuffles.  Ties go to the lower id because
// candidates arrive in ascending id order and only a strictly smaller distance displaces.
#include <mutex>

#include "common.cuh"
#include "knn_common.cuh"

namespace cpb {
namespace {

using knn::kFull;
using knn::bulk_g2s;
using knn::mbar_expect_tx;
using knn::mbar_init;
using knn::mbar_wait_bounded;
using knn::kWaitLimit;

// ---- SWAR component-mismatch count -------------------------------------------------------------
// Weighted form for residual codes (combined distance (h_primary << shift) + h_residual,
// include/cphnsw/core/types.hpp:284-302): a component of the first wp words of a row counts
// 1 + mul = 2^shift, the others 1.  CodeWeights{0, 0} is the plain count.
struct CodeWeights {
    uint32_t wp = 0, mul = 0;
};
template <bool U16>
struct FlagGroups {
    static constexpr int G = U16 ? 16 : 8;  // words whose flags fit one accumulator
};
// pm[g]: the flag bits of group g that belong to primary words.  Array word i holds the row's word
// 4 * (((i >> 2) + rot) & (WC / 4 - 1)) + (i & 3) (rot = 0: in order).
template <int WC, bool U16>
__device__ __forceinline__ void primary_masks(CodeWeights cw, int rot, uint32_t (&pm)[(WC + FlagGroups<U16>::G - 1) / FlagGroups<U16>::G]) {
    constexpr uint32_t HI = U16 ? 0x80008000u : 0x80808080u;
    constexpr int G = FlagGroups<U16>::G;
#pragma unroll
    for (int g = 0; g < (WC + G - 1) / G; ++g) pm[g] = 0;
#pragma unroll
    for (int w = 0; w < WC; ++w) {
        const uint32_t truew = 4u * (((w >> 2) + rot) & (WC / 4 - 1)) + (w & 3);
        if (truew < cw.wp) pm[w / G] |= HI >> (w % G);
    }
}

template <int WC, bool U16, bool WEIGHTED = true>
__device__ __forceinline__ uint32_t mismatch_count(const uint32_t (&a)[WC], const uint32_t (&b)[WC],
                                                   const uint32_t (&pm)[(WC + FlagGroups<U16>::G - 1) / FlagGroups<U16>::G],
                                                   uint32_t mul) {
    constexpr uint32_t LO = U16 ? 0x7fff7fffu : 0x7f7f7f7fu;
    constexpr uint32_t HI = ~LO;
    constexpr int G = FlagGroups<U16>::G;
    uint32_t d = 0;
#pragma unroll
    for (int g = 0; g < (WC + G - 1) / G; ++g) {
        uint32_t acc = 0;
#pragma unroll
        for (int w = g * G; w < WC && w < (g + 1) * G; ++w) {
            uint32_t x = a[w] ^ b[w];
            uint32_t t = (x & LO) + LO;  // top bit of each lane set iff its low bits are non-zero
            uint32_t y = t | x;          // ... or its own top bit is
            acc |= (y >> (w - g * G)) & (HI >> (w - g * G));
        }
        d += __popc(acc);
        if (WEIGHTED && mul) d += mul * __popc(acc & pm[g]);  // warp-uniform branch
    }
    return d;
}

// ---- pad [n][K] components to [n][WC] words ---------------------------------------------------------
__global__ void pad_codes_kernel(const uint8_t* __restrict__ src, uint64_t n, int row_bytes, int WC,
                                 uint32_t* __restrict__ dst) {
    uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    uint64_t total = n * uint64_t(WC);
    if (i >= total) return;
    uint64_t row = i / WC;
    int w = int(i % WC);
    uint32_t v = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        int off = 4 * w + b;
        if (off < row_bytes) v |= uint32_t(src[row * row_bytes + off]) << (8 * b);
    }
    dst[i] = v;
}

// ---- all-pairs distance matrix ---------------------------------------------------------------------
constexpr int kCdThreads = 256;
constexpr int kCdRowsA = 32;

template <int WC, bool U16>
__global__ void __launch_bounds__(kCdThreads)
code_distance_kernel(const uint32_t* __restrict__ a, uint64_t na, const uint32_t* __restrict__ b,
                     uint64_t nb, uint16_t* __restrict__ out, CodeWeights cwt) {
    uint32_t pm[(WC + FlagGroups<U16>::G - 1) / FlagGroups<U16>::G];
    primary_masks<WC, U16>(cwt, 0, pm);
    __shared__ uint32_t atile[kCdRowsA][WC];
    const uint64_t a0 = uint64_t(blockIdx.y) * kCdRowsA;
    const uint64_t j = uint64_t(blockIdx.x) * kCdThreads + threadIdx.x;
    const int rows = int(min(uint64_t(kCdRowsA), na - a0));
    for (int i = threadIdx.x; i < rows * WC; i += kCdThreads) (&atile[0][0])[i] = a[a0 * WC + i];
    __syncthreads();
    if (j >= nb) return;
    uint32_t mine[WC];
#pragma unroll
    for (int w = 0; w < WC; w += 4) {
        uint4 v = *reinterpret_cast<const uint4*>(b + j * WC + w);
        mine[w] = v.x;
        mine[w + 1] = v.y;
        mine[w + 2] = v.z;
        mine[w + 3] = v.w;
    }
    for (int i = 0; i < rows; ++i) {
        uint32_t other[WC];
#pragma unroll
        for (int w = 0; w < WC; ++w) other[w] = atile[i][w];
        out[(a0 + i) * nb + j] = uint16_t(mismatch_count<WC, U16>(other, mine, pm, cwt.mul));
    }
}

// ---- kNN graph ---------------------------------------------------------------------------------------
constexpr int kKnnWarps = 4;
constexpr int kKnnThreads = kKnnWarps * 32;
// candidates per shared-memory stage: 1024, or 512 for 128-byte rows (two stages must fit shared memory)
template <int WC>
struct KnnTile {
    static constexpr int value = WC == 32 ? knn::kTile / 2 : knn::kTile;
};

template <int WC, bool U16, int SLOTS, int Q, bool WEIGHTED>
__global__ void __launch_bounds__(kKnnThreads)
knn_graph_kernel(const uint32_t* __restrict__ codes, uint64_t n, uint32_t k, uint64_t row_begin,
                 uint64_t row_end, uint32_t* __restrict__ nbrs, uint16_t* __restrict__ dists,
                 uint32_t* __restrict__ status, uint32_t first_wait_polls, CodeWeights cwt) {
    constexpr int CH = WC / 4;  // 16-byte chunks per code row
    constexpr int CHLOG = CH == 1 ? 0 : (CH == 2 ? 1 : (CH == 4 ? 2 : 3));
    constexpr int kKnnTile = KnnTile<WC>::value;
    extern __shared__ __align__(128) unsigned char knn_smem[];
    uint4* stage0 = reinterpret_cast<uint4*>(knn_smem);
    uint4* stage1 = stage0 + size_t(kKnnTile) * CH;
    __shared__ uint64_t full_bar[2];
    __shared__ int abort_flag;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t tiles = (n + kKnnTile - 1) / kKnnTile;
    auto tile_bytes = [&](uint64_t t) -> uint32_t {
        uint64_t rows = min(uint64_t(kKnnTile), n - t * kKnnTile);
        return uint32_t(rows * WC * 4);
    };

    if (threadIdx.x == 0) {
        mbar_init(&full_bar[0], 1);
        mbar_init(&full_bar[1], 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint64_t t = 0; t < 2 && t < tiles; ++t) {
            mbar_expect_tx(&full_bar[t], tile_bytes(t));
            bulk_g2s(t == 0 ? stage0 : stage1, codes + t * kKnnTile * WC, tile_bytes(t), &full_bar[t]);
        }
    }

    // this warp's Q query rows, chunk order rotated per lane so that the shared-memory reads
    // of a quarter-warp fall into distinct banks
    const int rot = CH == 1 ? 0 : (lane >> (3 - CHLOG)) & (CH - 1);
    const uint64_t first_row = row_begin + (uint64_t(blockIdx.x) * kKnnWarps + warp) * Q;
    uint32_t pm[(WC + FlagGroups<U16>::G - 1) / FlagGroups<U16>::G];
    primary_masks<WC, U16>(cwt, rot, pm);
    uint32_t qw[Q][WC];
#pragma unroll
    for (int q = 0; q < Q; ++q) {
        uint64_t row = min(first_row + q, row_end - 1);
#pragma unroll
        for (int s = 0; s < CH; ++s) {
            int c = (s + rot) & (CH - 1);
            uint4 v = __ldg(reinterpret_cast<const uint4*>(codes + row * WC) + c);
            qw[q][4 * s] = v.x;
            qw[q][4 * s + 1] = v.y;
            qw[q][4 * s + 2] = v.z;
            qw[q][4 * s + 3] = v.w;
        }
    }
    // sorted running lists: element of rank (s*32 + lane) of row q
    uint32_t ld[Q][SLOTS], li[Q][SLOTS], tau[Q];
#pragma unroll
    for (int q = 0; q < Q; ++q) {
        tau[q] = kFull;
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            ld[q][s] = kFull;
            li[q][s] = kInvalidNode;
        }
    }

    bool lost = false;
    uint64_t lost_tile = 0;
    for (uint64_t t = 0; t < tiles; ++t) {
        const int st = int(t & 1);
        const uint32_t parity = uint32_t((t >> 1) & 1);
        if (!mbar_wait_bounded(&full_bar[st], parity, t == 0 ? first_wait_polls : kWaitLimit)) abort_flag = 1;
        __syncthreads();
        if (abort_flag) {
            lost = true;
            lost_tile = t;
            break;
        }
        const uint4* tile = st == 0 ? stage0 : stage1;
        const uint64_t base = t * kKnnTile;
        const int rows = int(min(uint64_t(kKnnTile), n - base));
        for (int c0 = 0; c0 < rows; c0 += 32) {
            const int c = c0 + lane;
            uint32_t cw[WC];
#pragma unroll
            for (int s = 0; s < CH; ++s) {
                uint4 v = tile[size_t(c) * CH + ((s + rot) & (CH - 1))];
                cw[4 * s] = v.x;
                cw[4 * s + 1] = v.y;
                cw[4 * s + 2] = v.z;
                cw[4 * s + 3] = v.w;
            }
            uint32_t d[Q];
            bool any = false;
#pragma unroll
            for (int q = 0; q < Q; ++q) {
                d[q] = c < rows ? mismatch_count<WC, U16, WEIGHTED>(qw[q], cw, pm, cwt.mul) : kFull;
                any |= d[q] < tau[q];
            }
            if (__any_sync(kFull, any)) {
#pragma unroll
                for (int q = 0; q < Q; ++q) {
                    uint32_t m = __ballot_sync(kFull, d[q] < tau[q]);
                    while (m) {
                        const int src = __ffs(m) - 1;
                        m &= m - 1;
                        const uint32_t dd = __shfl_sync(kFull, d[q], src);
                        if (dd >= tau[q]) continue;  // tightened by an earlier lane
                        const uint32_t id = uint32_t(base + c0 + src);
                        knn::list_insert<SLOTS>(ld[q], li[q], dd, id, lane);
                        tau[q] = knn::list_threshold<SLOTS>(ld[q], k);
                    }
                }
            }
        }
        __syncthreads();  // every warp is done with this stage
        if (threadIdx.x == 0 && t + 2 < tiles) {
            mbar_expect_tx(&full_bar[st], tile_bytes(t + 2));
            bulk_g2s(st == 0 ? stage0 : stage1, codes + (t + 2) * kKnnTile * WC, tile_bytes(t + 2),
                     &full_bar[st]);
        }
    }
    if (lost) {
        // report, then give copies still in flight a bounded chance to land before the block
        // (and its shared memory) goes away
        if (threadIdx.x == 0) {
            atomicExch(status, kStatusWaitTimeout);
            knn::drain_after_loss(full_bar, lost_tile, tiles);
        }
        return;
    }

    // write the rows out, dropping the row's own id
#pragma unroll
    for (int q = 0; q < Q; ++q) {
        const uint64_t row = first_row + q;
        if (row >= row_end) continue;
        knn::list_write<SLOTS>(ld[q], li[q], row, k, nbrs + (row - row_begin) * uint64_t(k),
                               dists ? dists + (row - row_begin) * uint64_t(k) : nullptr, lane);
    }
}

// ---- select_neighbors ----------------------------------------------------------------------------------
// SELECT-NEIGHBORS-HEURISTIC with keepPrunedConnections (resources/hnsw-paper/consolidated.tex:93-115):
// one warp per node; the kept set R lives in registers (member m on lane m%32, slot m/32), each
// candidate is tested against all of R in one step.
constexpr int kSelWarps = 4;
constexpr int kSelMaxK = 64;

template <int WC, bool U16>
__global__ void __launch_bounds__(kSelWarps * 32)
select_neighbors_kernel(const uint32_t* __restrict__ codes, uint64_t n, const uint32_t* __restrict__ cand, uint32_t k,
                        uint64_t row_begin, uint64_t row_end, uint32_t M, int keep_pruned,
                        uint32_t* __restrict__ adj, const uint32_t* __restrict__ row_ids, CodeWeights cwt) {
    // row_ids == nullptr: rows [row_begin, row_end), output row i at adj[i - row_begin];
    // otherwise rows row_ids[0 .. row_end - row_begin) and the output goes to adj[row] (in place)
    __shared__ uint32_t csm[kSelWarps][kSelMaxK][WC];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t slot = row_begin + uint64_t(blockIdx.x) * kSelWarps + warp;
    if (slot >= row_end) return;
    const uint64_t row = row_ids ? uint64_t(row_ids[slot - row_begin]) : slot;
    const uint32_t* crow = cand + (slot - row_begin) * uint64_t(k);
    uint32_t pm[(WC + FlagGroups<U16>::G - 1) / FlagGroups<U16>::G];
    primary_masks<WC, U16>(cwt, 0, pm);
    // candidate ids come from the caller: an id that names no code row counts as "no node"
    uint32_t cid[2];
    cid[0] = lane < int(k) ? crow[lane] : kInvalidNode;
    cid[1] = lane + 32 < int(k) ? crow[lane + 32] : kInvalidNode;
    if (cid[0] >= n) cid[0] = kInvalidNode;
    if (cid[1] >= n) cid[1] = kInvalidNode;
    uint32_t qc[WC];
#pragma unroll
    for (int w = 0; w < WC; w += 4) {
        uint4 v = __ldg(reinterpret_cast<const uint4*>(codes + row * WC + w));
        qc[w] = v.x, qc[w + 1] = v.y, qc[w + 2] = v.z, qc[w + 3] = v.w;
    }
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        const int t = lane + 32 * s;
        if (cid[s] != kInvalidNode) {
#pragma unroll
            for (int w = 0; w < WC; w += 4) {
                uint4 v = __ldg(reinterpret_cast<const uint4*>(codes + uint64_t(cid[s]) * WC + w));
                csm[warp][t][w] = v.x, csm[warp][t][w + 1] = v.y, csm[warp][t][w + 2] = v.z,
                csm[warp][t][w + 3] = v.w;
            }
        }
    }
    __syncwarp();

    uint32_t rc[2][WC];
    uint32_t rsize = 0;
    unsigned long long kept = 0, disc = 0;
    for (uint32_t t = 0; t < k && rsize < M; ++t) {
        const uint32_t e = __shfl_sync(kFull, t < 32 ? cid[0] : cid[1], int(t & 31));
        if (e == kInvalidNode) continue;
        uint32_t ec[WC];
#pragma unroll
        for (int w = 0; w < WC; ++w) ec[w] = csm[warp][t][w];
        const uint32_t d_eq = mismatch_count<WC, U16>(ec, qc, pm, cwt.mul);
        bool viol = false;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const uint32_t m = uint32_t(lane + 32 * s);
            if (m < rsize) viol |= !(d_eq < mismatch_count<WC, U16>(ec, rc[s], pm, cwt.mul));
        }
        if (__any_sync(kFull, viol)) {
            disc |= 1ull << t;
        } else {
            kept |= 1ull << t;
#pragma unroll
            for (int s = 0; s < 2; ++s)
                if (uint32_t(lane + 32 * s) == rsize) {
#pragma unroll
                    for (int w = 0; w < WC; ++w) rc[s][w] = ec[w];
                }
            ++rsize;
        }
    }
    uint32_t* out = adj + (row_ids ? row : slot - row_begin) * uint64_t(M);
    const uint32_t n_disc = keep_pruned ? uint32_t(__popcll(disc)) : 0u;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        const int t = lane + 32 * s;
        const unsigned long long below = (1ull << t) - 1ull;
        uint32_t pos = kInvalidNode;
        if ((kept >> t) & 1ull) pos = uint32_t(__popcll(kept & below));
        else if (keep_pruned && ((disc >> t) & 1ull)) pos = rsize + uint32_t(__popcll(disc & below));
        if (pos < M) out[pos] = cid[s];
    }
    const uint32_t total = min(M, rsize + n_disc);
    for (uint32_t o = total + lane; o < M; o += 32) out[o] = kInvalidNode;
}

// ---- reverse edges of an incremental insertion ---------------------------------------------------------------
// New nodes (ids >= n_old) have chosen their neighbours among the old nodes; every old node v that
// was chosen gets the choosers as candidates for its own row.
// in-degree of every old node from the new rows
__global__ void rev_count_kernel(const uint32_t* __restrict__ new_adj, uint64_t m, int M, uint64_t n_old,
                                 uint32_t* __restrict__ cnt) {
    const uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= m * M) return;
    const uint32_t v = new_adj[t];
    if (v < n_old) atomicAdd(cnt + v, 1u);
}
// a segment of the incoming list for every old node with incoming edges; the list of those nodes
// (counters[0] = entries used in the incoming list, counters[1] = affected nodes)
__global__ void rev_alloc_kernel(const uint32_t* __restrict__ cnt, uint64_t n_old, uint32_t* __restrict__ seg,
                                 uint32_t* __restrict__ aff, uint32_t* __restrict__ counters) {
    const uint64_t v = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (v >= n_old || cnt[v] == 0) return;
    seg[v] = atomicAdd(counters, cnt[v]);
    aff[atomicAdd(counters + 1, 1u)] = uint32_t(v);
}
__global__ void rev_fill_kernel(const uint32_t* __restrict__ new_adj, uint64_t m, int M, uint64_t n_old,
                                const uint32_t* __restrict__ seg, uint32_t* __restrict__ fill, uint32_t* __restrict__ inc) {
    const uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= m * M) return;
    const uint32_t v = new_adj[t];
    if (v < n_old) inc[seg[v] + atomicAdd(fill + v, 1u)] = uint32_t(n_old + t / M);
}
// One warp per affected old node v: its current neighbours and the new nodes that chose it, the 64
// closest to v by (code distance, id) in ascending order -> cand_out[i][64] (the order in which
// the incoming list was filled does not matter).
template <int WC, bool U16>
__global__ void __launch_bounds__(kSelWarps * 32)
rev_merge_kernel(const uint32_t* __restrict__ codes, uint64_t n, const uint32_t* __restrict__ adj, int M,
                 const uint32_t* __restrict__ aff, uint32_t n_aff, const uint32_t* __restrict__ cnt,
                 const uint32_t* __restrict__ seg, const uint32_t* __restrict__ inc, uint32_t* __restrict__ cand_out,
                 CodeWeights cwt) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t i = blockIdx.x * kSelWarps + warp;
    if (i >= n_aff) return;
    uint32_t pm[(WC + FlagGroups<U16>::G - 1) / FlagGroups<U16>::G];
    primary_masks<WC, U16>(cwt, 0, pm);
    const uint32_t v = aff[i];
    uint32_t qc[WC];
#pragma unroll
    for (int w = 0; w < WC; w += 4) {
        const uint4 c = __ldg(reinterpret_cast<const uint4*>(codes + uint64_t(v) * WC + w));
        qc[w] = c.x, qc[w + 1] = c.y, qc[w + 2] = c.z, qc[w + 3] = c.w;
    }
    uint32_t ld[2] = {kFull, kFull}, li[2] = {kInvalidNode, kInvalidNode};
    const uint32_t total = uint32_t(M) + cnt[v];
    for (uint32_t c0 = 0; c0 < total; c0 += 32) {
        const uint32_t c = c0 + lane;
        uint32_t w = kInvalidNode;
        if (c < uint32_t(M)) w = adj[uint64_t(v) * M + c];
        else if (c < total) w = inc[seg[v] + (c - M)];
        if (w >= n) w = kInvalidNode;  // rows installed or loaded from outside may hold anything
        uint32_t dd = kFull;
        if (w != kInvalidNode) {
            uint32_t wc[WC];
#pragma unroll
            for (int x = 0; x < WC; x += 4) {
                const uint4 cc = __ldg(reinterpret_cast<const uint4*>(codes + uint64_t(w) * WC + x));
                wc[x] = cc.x, wc[x + 1] = cc.y, wc[x + 2] = cc.z, wc[x + 3] = cc.w;
            }
            dd = mismatch_count<WC, U16>(wc, qc, pm, cwt.mul);
        }
        uint32_t live = __ballot_sync(kFull, w != kInvalidNode);
        while (live) {
            const int src = __ffs(live) - 1;
            live &= live - 1;
            const uint32_t d1 = __shfl_sync(kFull, dd, src), w1 = __shfl_sync(kFull, w, src);
            // rank = members below (d1, w1); whatever moves past place 63 falls off
            int p = 0;
#pragma unroll
            for (int s = 0; s < 2; ++s) p += __popc(__ballot_sync(kFull, ld[s] < d1 || (ld[s] == d1 && li[s] < w1)));
            if (p >= 64) continue;
#pragma unroll
            for (int s = 1; s >= 0; --s) {
                uint32_t ud = __shfl_up_sync(kFull, ld[s], 1), ui = __shfl_up_sync(kFull, li[s], 1);
                if (s > 0) {
                    const uint32_t cd = __shfl_sync(kFull, ld[s - 1], 31), ci = __shfl_sync(kFull, li[s - 1], 31);
                    if (lane == 0) ud = cd, ui = ci;
                }
                const int rank = s * 32 + lane;
                if (rank > p) ld[s] = ud, li[s] = ui;
                else if (rank == p) ld[s] = d1, li[s] = w1;
            }
        }
    }
    cand_out[uint64_t(i) * 64 + lane] = li[0];
    cand_out[uint64_t(i) * 64 + 32 + lane] = li[1];
}

// ---- host-side dispatch ----------------------------------------------------------------------------------
struct PaddedCodes {
    const uint32_t* p = nullptr;
};

// Returns a [n][WC]-word view of the codes: the caller's buffer when rows are already WC words,
// else a zero-padded copy in `scratch`.
int padded_view(cphnsw_b200_index* h, const void* d_codes, uint64_t n, int WC, DevBuf& scratch,
                cudaStream_t st, const uint32_t** out) {
    const int row_bytes = int(h->K * h->comp_bytes);
    if ((reinterpret_cast<uintptr_t>(d_codes) & 15) != 0 && row_bytes == WC * 4) {
        set_error("device code buffer must be 16-byte aligned");
        return CPHNSW_B200_E_INVALID;
    }
    if (row_bytes == WC * 4) {
        *out = static_cast<const uint32_t*>(d_codes);
        return 0;
    }
    CPB_TRY(scratch.reserve(size_t(n) * WC * 4 + 16));
    uint64_t total = n * uint64_t(WC);
    if (total) {
        pad_codes_kernel<<<unsigned((total + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t*>(d_codes), n,
                                                                        row_bytes, WC, scratch.as<uint32_t>());
        h->launches++;
        CPB_CUDA(cudaGetLastError());
    }
    *out = scratch.as<uint32_t>();
    return 0;
}

}  // namespace

// weights of the handle's code distance (plain unless residual bits are set)
static CodeWeights code_weights(const cphnsw_b200_index* h) {
    CodeWeights w;
    if (h->residual_bits) {
        w.wp = (h->K - h->residual_bits) * h->comp_bytes / 4;
        w.mul = (1u << h->residual_shift) - 1u;
    }
    return w;
}

int code_row_words(uint32_t K, uint32_t comp_bytes) {
    uint32_t bytes = K * comp_bytes;
    if (bytes <= 16) return 4;
    if (bytes <= 32) return 8;
    if (bytes <= 64) return 16;
    if (bytes <= 128) return 32;
    return 0;
}

#define CPB_DISPATCH_WC(WCV, U16V, CALL)                                   \
    do {                                                                   \
        if (WCV == 4 && !(U16V)) { CALL(4, false); }                       \
        else if (WCV == 4) { CALL(4, true); }                              \
        else if (WCV == 8 && !(U16V)) { CALL(8, false); }                  \
        else if (WCV == 8) { CALL(8, true); }                              \
        else if (WCV == 16 && !(U16V)) { CALL(16, false); }                \
        else if (WCV == 16) { CALL(16, true); }                            \
        else if (!(U16V)) { CALL(32, false); }                             \
        else { CALL(32, true); }                                           \
    } while (0)

int launch_code_distance(cphnsw_b200_index* h, const void* d_a, uint64_t na, const void* d_b, uint64_t nb,
                         uint16_t* d_out, cudaStream_t st) {
    if (na == 0 || nb == 0) return 0;
    const int WC = code_row_words(h->K, h->comp_bytes);
    if (!WC) {
        set_error("code rows wider than 128 bytes are not supported by the distance kernels (K*component_bytes=%u)",
                  h->K * h->comp_bytes);
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    const bool u16 = h->comp_bytes == 2;
    const uint32_t *pa, *pb;
    CPB_TRY(padded_view(h, d_a, na, WC, h->s_pad, st, &pa));
    CPB_TRY(padded_view(h, d_b, nb, WC, h->s_pad2, st, &pb));
    dim3 grid(unsigned((nb + kCdThreads - 1) / kCdThreads), unsigned((na + kCdRowsA - 1) / kCdRowsA));
    LaunchTimer timer(h, kKernelCodeDistance, st);
    const CodeWeights cwt = code_weights(h);
#define CALL(W, U) code_distance_kernel<W, U><<<grid, kCdThreads, 0, st>>>(pa, na, pb, nb, d_out, cwt)
    CPB_DISPATCH_WC(WC, u16, CALL);
#undef CALL
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

template <int WC, bool U16, int SLOTS, int Q, bool WEIGHTED>
static int launch_knn_w(cphnsw_b200_index* h, const uint32_t* codes, uint64_t n, uint32_t k, uint64_t rb,
                        uint64_t re, uint32_t* nbrs, uint16_t* dist, cudaStream_t st) {
    const size_t smem = size_t(2) * KnnTile<WC>::value * WC * 4;
    auto kernel = knn_graph_kernel<WC, U16, SLOTS, Q, WEIGHTED>;
    CPB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    const uint64_t rows = re - rb;
    const uint64_t blocks = (rows + kKnnWarps * Q - 1) / (kKnnWarps * Q);
    LaunchTimer timer(h, kKernelKnn, st);
    kernel<<<unsigned(blocks), kKnnThreads, smem, st>>>(codes, n, k, rb, re, nbrs, dist, h->d_status.as<uint32_t>(), h->first_wait_polls,
                                                       code_weights(h));
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

// the weighted (residual-code) distance is a separate instantiation: the plain count pays nothing for it
template <int WC, bool U16, int SLOTS, int Q>
static int launch_knn_t(cphnsw_b200_index* h, const uint32_t* codes, uint64_t n, uint32_t k, uint64_t rb,
                        uint64_t re, uint32_t* nbrs, uint16_t* dist, cudaStream_t st) {
    if (h->residual_bits) return launch_knn_w<WC, U16, SLOTS, Q, true>(h, codes, n, k, rb, re, nbrs, dist, st);
    return launch_knn_w<WC, U16, SLOTS, Q, false>(h, codes, n, k, rb, re, nbrs, dist, st);
}

template <int WC, bool U16>
static int launch_knn_slots(cphnsw_b200_index* h, const uint32_t* codes, uint64_t n, uint32_t k, uint64_t rb,
                            uint64_t re, uint32_t* nbrs, uint16_t* dist, cudaStream_t st) {
    constexpr int Q = WC == 32 ? 2 : (WC == 16 ? 4 : 8);
    const uint32_t need = k + 1;  // the row's own id may occupy one place
    if (need <= 64) return launch_knn_t<WC, U16, 2, Q>(h, codes, n, k, rb, re, nbrs, dist, st);
    if (need <= 96) return launch_knn_t<WC, U16, 3, Q>(h, codes, n, k, rb, re, nbrs, dist, st);
    return launch_knn_t<WC, U16, 4, Q>(h, codes, n, k, rb, re, nbrs, dist, st);
}

int launch_knn_graph(cphnsw_b200_index* h, const void* d_codes, uint64_t n, uint32_t k, uint64_t row_begin,
                     uint64_t row_end, uint32_t* d_nbrs, uint16_t* d_dist, cudaStream_t st) {
    if (row_end <= row_begin) return 0;
    if (k == 0 || k > 127) {
        set_error("knn_graph: k must be in 1..127 (got %u)", k);
        return CPHNSW_B200_E_INVALID;
    }
    if (row_end > n) {
        set_error("knn_graph: row range [%llu,%llu) exceeds n=%llu", (unsigned long long)row_begin,
                  (unsigned long long)row_end, (unsigned long long)n);
        return CPHNSW_B200_E_INVALID;
    }
    const int WC = code_row_words(h->K, h->comp_bytes);
    if (!WC) {
        set_error("code rows wider than 128 bytes are not supported by the distance kernels");
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    if (h->knn_kernel == 2 && !knn_sliced_supported(h)) {
        set_error("knn_kernel=2 (bit-sliced) needs K = 16, 32 or 64 with uint8 components, K = 16 / 32 with padded dim 1024, or one-byte sign-bit codes of whole blocks of 8 components (K <= 120)");
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    if (h->knn_kernel != 1 && knn_sliced_supported(h))
        return launch_knn_graph_sliced(h, d_codes, n, k, row_begin, row_end, d_nbrs, d_dist, st);
    const bool u16 = h->comp_bytes == 2;
    const uint32_t* pc;
    CPB_TRY(padded_view(h, d_codes, n, WC, h->s_pad, st, &pc));
#define CALL(W, U) return launch_knn_slots<W, U>(h, pc, n, k, row_begin, row_end, d_nbrs, d_dist, st)
    CPB_DISPATCH_WC(WC, u16, CALL);
#undef CALL
    return 0;
}

int launch_select_neighbors(cphnsw_b200_index* h, const void* d_codes, uint64_t n, const uint32_t* d_cand,
                            uint32_t k, uint64_t row_begin, uint64_t row_end, uint32_t M, int keep_pruned,
                            uint32_t* d_adj, cudaStream_t st, const uint32_t* d_row_ids) {
    if (row_end <= row_begin) return 0;
    if (k == 0 || k > kSelMaxK || M == 0 || M > 64) {
        set_error("select_neighbors: need 1 <= k <= 64 and 1 <= M <= 64 (got k=%u M=%u)", k, M);
        return CPHNSW_B200_E_INVALID;
    }
    const int WC = code_row_words(h->K, h->comp_bytes);
    if (!WC) {
        set_error("code rows wider than 128 bytes are not supported by the distance kernels");
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    const bool u16 = h->comp_bytes == 2;
    const uint32_t* pc;
    CPB_TRY(padded_view(h, d_codes, n, WC, h->s_pad, st, &pc));
    const uint64_t rows = row_end - row_begin;
    const unsigned grid = unsigned((rows + kSelWarps - 1) / kSelWarps);
    LaunchTimer timer(h, kKernelSelect, st);
    const CodeWeights cwt = code_weights(h);
#define CALL(W, U)                                                                                          \
    select_neighbors_kernel<W, U><<<grid, kSelWarps * 32, 0, st>>>(pc, n, d_cand, k, row_begin, row_end, M, \
                                                                   keep_pruned, d_adj, d_row_ids, cwt)
    CPB_DISPATCH_WC(WC, u16, CALL);
#undef CALL
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

// Reverse edges after the rows [n_old, n_old + m) of d_adj have been chosen among the old nodes:
// every old node with incoming new edges re-selects its row from (current row + choosers).
int launch_reverse_edges(cphnsw_b200_index* h, const void* d_codes, uint64_t n_old, uint64_t m, uint32_t* d_adj,
                         uint32_t M, int keep_pruned, cudaStream_t st) {
    if (m == 0 || n_old == 0) return 0;
    const int WC = code_row_words(h->K, h->comp_bytes);
    if (!WC) {
        set_error("code rows wider than 128 bytes are not supported by the distance kernels");
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    const bool u16 = h->comp_bytes == 2;
    const uint64_t edges = m * M;
    // scratch: cnt, seg, fill [n_old]; aff [n_old]; inc [edges]
    CPB_TRY(h->s_in.reserve((size_t(n_old) * 4 + edges) * 4 + 64));
    uint32_t* cnt = h->s_in.as<uint32_t>();
    uint32_t* seg = cnt + n_old;
    uint32_t* fill = seg + n_old;
    uint32_t* aff = fill + n_old;
    uint32_t* inc = aff + n_old;
    uint32_t* counters = h->d_status.as<uint32_t>() + 6;  // two words
    CPB_CUDA(cudaMemsetAsync(cnt, 0, size_t(n_old) * 4, st));
    CPB_CUDA(cudaMemsetAsync(fill, 0, size_t(n_old) * 4, st));
    CPB_CUDA(cudaMemsetAsync(counters, 0, 8, st));
    const uint32_t* new_adj = d_adj + n_old * M;
    rev_count_kernel<<<unsigned((edges + 255) / 256), 256, 0, st>>>(new_adj, m, int(M), n_old, cnt);
    rev_alloc_kernel<<<unsigned((n_old + 255) / 256), 256, 0, st>>>(cnt, n_old, seg, aff, counters);
    rev_fill_kernel<<<unsigned((edges + 255) / 256), 256, 0, st>>>(new_adj, m, int(M), n_old, seg, fill, inc);
    h->launches += 3;
    CPB_CUDA(cudaGetLastError());
    uint32_t host_counters[2] = {0, 0};
    CPB_CUDA(cudaMemcpyAsync(host_counters, counters, 8, cudaMemcpyDeviceToHost, st));
    CPB_CUDA(cudaStreamSynchronize(st));
    const uint32_t n_aff = host_counters[1];
    if (n_aff == 0) return 0;
    CPB_TRY(h->s_in2.reserve(size_t(n_aff) * 64 * 4 + 16));
    uint32_t* cand = h->s_in2.as<uint32_t>();
    const uint32_t* pc;
    CPB_TRY(padded_view(h, d_codes, n_old + m, WC, h->s_pad, st, &pc));
    const unsigned grid = (n_aff + kSelWarps - 1) / kSelWarps;
    const CodeWeights cwt = code_weights(h);
#define CALL(W, U) rev_merge_kernel<W, U><<<grid, kSelWarps * 32, 0, st>>>(pc, n_old + m, d_adj, int(M), aff, n_aff, cnt, seg, inc, cand, cwt)
    CPB_DISPATCH_WC(WC, u16, CALL);
#undef CALL
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return launch_select_neighbors(h, d_codes, n_old + m, cand, 64, 0, n_aff, M, keep_pruned, d_adj, st, aff);
}

}  // namespace cpb

// ---- allocation-free code distance -------------------------------------------------------------------
// For callers that must not allocate device memory (see the declaration in cphnsw_b200.h).
// The padded copies of both operands, which the ordinary entry point keeps in buffers it
// allocates on demand, live here in one statically sized device array that is part of the
// loaded module on every GPU that loads the library.
namespace {

constexpr size_t kNoAllocScratchBytes = size_t(1) << 20;  // padded copies of A and B together
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mutex;
uint32_t* g_noalloc_ptr[kNoAllocMaxDevices] = {};  // device address of the array, per device

// `g_noalloc_scratch` in host code is only a stand-in for the symbol; the address a kernel can
// use has to be asked for, once per device, with that device current.
int noalloc_scratch(uint32_t** out) {
    int dev = -1;
    CPB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kNoAllocMaxDevices) {
        cpb::set_error("code_distance_noalloc: device ordinal %d not supported", dev);
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        CPB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_noalloc_ptr[dev] = static_cast<uint32_t*>(p);
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}

}  // namespace

extern "C" int cphnsw_b200_code_distance_noalloc(const void* d_a, uint64_t na, const void* d_b, uint64_t nb,
                                                 uint32_t K, uint32_t component_bytes, uint16_t* d_out,
                                                 void* stream) {
    using namespace cpb;
    if (K == 0 || K > 256 || (component_bytes != 1 && component_bytes != 2)) {
        set_error("code_distance_noalloc: need 1 <= K <= 256 and component_bytes 1 or 2");
        return CPHNSW_B200_E_INVALID;
    }
    if (na == 0 || nb == 0) return 0;
    if (!d_a || !d_b || !d_out) {
        set_error("code_distance_noalloc: null pointer");
        return CPHNSW_B200_E_INVALID;
    }
    const int WC = code_row_words(K, component_bytes);
    if (!WC) {
        set_error("code_distance_noalloc: code rows wider than 128 bytes are not supported (K*component_bytes=%u)",
                  K * component_bytes);
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    const uint64_t capacity_rows = kNoAllocScratchBytes / (uint64_t(WC) * 4);
    if (na > capacity_rows || nb > capacity_rows || na + nb > capacity_rows) {
        set_error("code_distance_noalloc: na + nb = %llu rows exceed the built-in scratch (%llu rows of %d bytes = %zu bytes); "
                  "split the call or use cphnsw_b200_code_distance_dev",
                  (unsigned long long)(na + nb), (unsigned long long)capacity_rows, WC * 4, kNoAllocScratchBytes);
        return CPHNSW_B200_E_INVALID;
    }
    uint32_t* scratch = nullptr;
    CPB_TRY(noalloc_scratch(&scratch));
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t* pa = scratch;
    uint32_t* pb = scratch + na * WC;  // na*WC*4 is a multiple of 16: the 128-bit loads stay aligned
    const int row_bytes = int(K * component_bytes);
    // every word of both padded copies is rewritten here, so nothing left by an earlier call is read
    pad_codes_kernel<<<unsigned((na * WC + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t*>(d_a), na, row_bytes, WC, pa);
    pad_codes_kernel<<<unsigned((nb * WC + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t*>(d_b), nb, row_bytes, WC, pb);
    const bool u16 = component_bytes == 2;
    dim3 grid(unsigned((nb + kCdThreads - 1) / kCdThreads), unsigned((na + kCdRowsA - 1) / kCdRowsA));
#define CALL(W, U) code_distance_kernel<W, U><<<grid, kCdThreads, 0, st>>>(pa, na, pb, nb, d_out, CodeWeights{})
    CPB_DISPATCH_WC(WC, u16, CALL);
#undef CALL
    CPB_CUDA(cudaGetLastError());
    return 0;
}
