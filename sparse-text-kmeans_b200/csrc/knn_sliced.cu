// Brute-force code-distance kNN graph with a bit-sliced distance (K = 16, 32 or 64; uint8 components,
// uint16 components of an 11-bit code, i.e. padded dim 1024 (K = 16 or 32), or sign-bit codes of the
// binary-code mode: one plane per component).
//
// Same result as knn_graph_kernel in distance.cu (k smallest under (distance, id), self excluded),
// four times fewer integer instructions per pair.  The candidates are re-laid out once, 32 at a
// time, as bit planes: word (r, b) of a group holds bit b of component r of its 32 candidates.
// For a query with component q_r, the candidates that differ from it in rotation r are
//      neq_r = OR_b ( plane(r,b) XOR mask(q_r,b) ),      mask = all ones if bit b of q_r is set,
// one 3-input logic instruction per bit plane (8 or 11 per rotation) for 32 candidates; the K one-bit planes neq_r are then summed
// with carry-save adders (two logic instructions per full adder, K - 6 adders for K = 32) into
// six planes holding the 32 distances, which are compared with the row's admission threshold in
// bit-sliced form as well.  Only candidates below the threshold (rare once the list has warmed
// up) are unpacked and inserted into the row's running list.
//
// Work split: a warp owns Q query rows; their masks (1 KB each at K = 32) sit in shared memory
// and are read with broadcast 128-bit loads.  A tile is 1024 candidates = 32 groups, one group
// per lane, laid out [16-byte chunk][group] so that the lanes' 128-bit loads are conflict-free;
// tiles arrive by bulk asynchronous copies (two stages, bounded waits), as in the byte-wise kernel.
#include <utility>

#include "knn_common.cuh"

namespace cpb {
namespace {

using knn::kFull;
constexpr int kSlWarps = 4;
constexpr int kSlQ = 8;  // query rows per warp

// compile-time loop: calls f(integral_constant<int, 0>), ..., f(integral_constant<int, N-1>)
template <class F, int... Is>
__device__ __forceinline__ void static_for_impl(F&& f, std::integer_sequence<int, Is...>) {
    (f(std::integral_constant<int, Is>{}), ...);
}
template <int N, class F>
__device__ __forceinline__ void static_for(F&& f) {
    static_for_impl(static_cast<F&&>(f), std::make_integer_sequence<int, N>{});
}

// full adder on bit planes: (carry, sum) of a + b + c
__device__ __forceinline__ void csa(uint32_t& carry, uint32_t& sum, uint32_t a, uint32_t b, uint32_t c) {
    const uint32_t u = a ^ b;
    carry = (a & b) | (u & c);
    sum = u ^ c;
}

// ---- layout transform: codes [n][K] components -> tiles [tile][chunk (K*NB/4)][group (32)][4 words] --
// one warp per group of 32 candidates; plane index w = r*NB + b; candidates past n read as zero
// codes (masked out later)
template <typename CompT>
__global__ void slice_codes_kernel(const CompT* __restrict__ codes, uint64_t n, int K, int NB,
                                   uint32_t* __restrict__ out, uint64_t n_groups) {
    const int lane = threadIdx.x & 31;
    const uint64_t g = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (g >= n_groups) return;
    const uint64_t cand = g * 32 + lane;
    const uint64_t tile = g >> 5;
    const int group = int(g & 31);
    const int words_per_group = K * NB;  // bit planes per group
    uint32_t* tile_out = out + tile * uint64_t(words_per_group) * 32;
    for (int r = 0; r < K; ++r) {
        const uint32_t comp = cand < n ? uint32_t(codes[cand * K + r]) : 0u;
        for (int b = 0; b < NB; ++b) {
            const uint32_t plane = __ballot_sync(kFull, (comp >> b) & 1u);
            const int w = r * NB + b;  // chunk = w / 4, word in chunk = w % 4
            if (lane == (w & 31)) tile_out[(size_t(w >> 2) * 32 + group) * 4 + (w & 3)] = plane;
        }
    }
}

template <typename CompT, int NB, int NBLK, int SLOTS, int WARPS>  // NB bit planes per component, NBLK = K / 8
__global__ void __launch_bounds__(WARPS * 32)
knn_sliced_kernel(const uint32_t* __restrict__ sliced, const CompT* __restrict__ codes, uint64_t n, uint32_t k,
                  uint64_t row_begin, uint64_t row_end, uint32_t* __restrict__ nbrs, uint16_t* __restrict__ dists,
                  uint32_t* __restrict__ status, uint32_t first_wait_polls) {
    constexpr int K = NBLK * 8;
    constexpr int CHUNKS = K * NB / 4;             // 16-byte chunks per group
    constexpr uint32_t TILE_BYTES = CHUNKS * 32 * 16;
    extern __shared__ __align__(128) unsigned char sl_smem[];
    uint4* stage0 = reinterpret_cast<uint4*>(sl_smem);
    uint4* stage1 = stage0 + CHUNKS * 32;
    uint4* masks = stage1 + CHUNKS * 32;           // [warp][q][chunk]
    __shared__ uint64_t full_bar[2];
    __shared__ int abort_flag;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t tiles = (n + knn::kTile - 1) / knn::kTile;

    if (threadIdx.x == 0) {
        knn::mbar_init(&full_bar[0], 1);
        knn::mbar_init(&full_bar[1], 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint64_t t = 0; t < 2 && t < tiles; ++t) {
            knn::mbar_expect_tx(&full_bar[t], TILE_BYTES);
            knn::bulk_g2s(t == 0 ? stage0 : stage1, sliced + t * (TILE_BYTES / 4), TILE_BYTES, &full_bar[t]);
        }
    }

    // masks of this warp's Q rows: word (r, b) is all ones when bit b of the row's component r is set
    const uint64_t first_row = row_begin + (uint64_t(blockIdx.x) * WARPS + warp) * kSlQ;
    uint4* my_masks = masks + size_t(warp) * kSlQ * CHUNKS;
    for (int q = 0; q < kSlQ; ++q) {
        const uint64_t row = min(first_row + q, row_end - 1);
        uint32_t* mw = reinterpret_cast<uint32_t*>(my_masks + q * CHUNKS);
        for (int w = lane; w < K * NB; w += 32) {
            const uint32_t comp = uint32_t(codes[row * K + w / NB]);
            mw[w] = ((comp >> (w % NB)) & 1u) ? kFull : 0u;
        }
    }
    __syncwarp();

    uint32_t ld[kSlQ][SLOTS], li[kSlQ][SLOTS], tau[kSlQ];
#pragma unroll
    for (int q = 0; q < kSlQ; ++q) {
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
        if (!knn::mbar_wait_bounded(&full_bar[st], parity, t == 0 ? first_wait_polls : knn::kWaitLimit)) abort_flag = 1;
        __syncthreads();
        if (abort_flag) {
            lost = true;
            lost_tile = t;
            break;
        }
        const uint4* tile = st == 0 ? stage0 : stage1;
        const uint64_t group_base = t * knn::kTile + uint64_t(lane) * 32;  // id of this lane's first candidate
        // candidates of this lane's group that exist
        const uint32_t valid = group_base >= n ? 0u : (n - group_base >= 32 ? kFull : ((1u << (n - group_base)) - 1u));

        // distance planes of the Q rows against this lane's 32 candidates
        uint32_t ones[kSlQ], twos[kSlQ], fours[kSlQ], eights[kSlQ], sixteens[kSlQ], thirtytwos[kSlQ], sixtyfours[kSlQ];
        uint32_t pend8[kSlQ], pend16[kSlQ];
#pragma unroll
        for (int q = 0; q < kSlQ; ++q)
            ones[q] = twos[q] = fours[q] = eights[q] = sixteens[q] = thirtytwos[q] = sixtyfours[q] = pend8[q] = pend16[q] = 0;

#pragma unroll 1
        for (int blk = 0; blk < NBLK; ++blk) {
            uint32_t twosA[kSlQ], twosB[kSlQ], foursA[kSlQ], foursB[kSlQ], prev[kSlQ], x[kSlQ];
            // the 8 rotations of this block span 8*NB planes = 2*NB chunks; the chunk index is a
            // compile-time constant so that every plane's (rotation, bit) is resolved statically
            static_for<2 * NB>([&](auto cc) {
                constexpr int c = decltype(cc)::value;
                const int chunk = blk * 2 * NB + c;
                const uint4 s4 = tile[size_t(chunk) * 32 + lane];
                const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int q = 0; q < kSlQ; ++q) {
                    const uint4 m4 = my_masks[q * CHUNKS + chunk];
                    const uint32_t mw[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int widx = c * 4 + i;  // plane within the block
                        const int rr = widx / NB;    // rotation within the block (0..7)
                        const int b = widx % NB;     // bit of the component
                        const uint32_t t = sw[i] ^ mw[i];
                        x[q] = b == 0 ? t : (x[q] | t);
                        if (b == NB - 1) {
                            // carry-save accumulation of this rotation's "differs" plane
                            if (rr & 1) {
                                uint32_t& tw = (rr & 2) ? twosB[q] : twosA[q];
                                csa(tw, ones[q], ones[q], prev[q], x[q]);
                                if ((rr & 3) == 3) {
                                    uint32_t& fo = (rr & 4) ? foursB[q] : foursA[q];
                                    csa(fo, twos[q], twos[q], twosA[q], twosB[q]);
                                    if (rr == 7) {
                                        uint32_t e8;
                                        csa(e8, fours[q], fours[q], foursA[q], foursB[q]);
                                        if (NBLK == 8) {
                                            // 64 rotations: the weight-8 carry of every block ripples into the
                                            // 8 / 16 / 32 / 64 planes
                                            const uint32_t c16 = eights[q] & e8;
                                            eights[q] ^= e8;
                                            const uint32_t c32 = sixteens[q] & c16;
                                            sixteens[q] ^= c16;
                                            const uint32_t c64 = thirtytwos[q] & c32;
                                            thirtytwos[q] ^= c32;
                                            sixtyfours[q] ^= c64;
                                        } else if (blk & 1) {
                                            uint32_t s16;
                                            csa(s16, eights[q], eights[q], pend8[q], e8);
                                            if (NBLK == 2) {
                                                sixteens[q] = s16;
                                            } else if (blk & 2) {
                                                csa(thirtytwos[q], sixteens[q], sixteens[q], pend16[q], s16);
                                            } else {
                                                pend16[q] = s16;
                                            }
                                        } else {
                                            pend8[q] = e8;
                                        }
                                    }
                                }
                            } else {
                                prev[q] = x[q];
                            }
                        }
                    }
                }
            });
        }

#pragma unroll
        for (int q = 0; q < kSlQ; ++q) {
            // candidates with distance < tau[q], bit-sliced compare against the warp-uniform threshold
            uint32_t pass;
            if (tau[q] > uint32_t(K)) {
                pass = kFull;
            } else {
                const uint32_t plane[7] = {ones[q], twos[q], fours[q], eights[q], sixteens[q], thirtytwos[q], sixtyfours[q]};
                uint32_t lt = 0, eq = kFull;
#pragma unroll
                for (int b = (NBLK == 8 ? 6 : 5); b >= 0; --b) {
                    if ((tau[q] >> b) & 1u) {
                        lt |= eq & ~plane[b];
                        eq &= plane[b];
                    } else {
                        eq &= ~plane[b];
                    }
                }
                pass = lt;
            }
            pass &= valid;
            uint32_t lanes = __ballot_sync(kFull, pass != 0);
            while (lanes) {
                const int src = __ffs(lanes) - 1;
                lanes &= lanes - 1;
                uint32_t pm = __shfl_sync(kFull, pass, src);
                const uint32_t p0 = __shfl_sync(kFull, ones[q], src), p1 = __shfl_sync(kFull, twos[q], src),
                               p2 = __shfl_sync(kFull, fours[q], src), p3 = __shfl_sync(kFull, eights[q], src),
                               p4 = __shfl_sync(kFull, sixteens[q], src), p5 = __shfl_sync(kFull, thirtytwos[q], src),
                               p6 = NBLK == 8 ? __shfl_sync(kFull, sixtyfours[q], src) : 0u;
                const uint64_t src_base = t * knn::kTile + uint64_t(src) * 32;
                while (pm) {
                    const int bit = __ffs(pm) - 1;
                    pm &= pm - 1;
                    const uint32_t dd = ((p0 >> bit) & 1u) | (((p1 >> bit) & 1u) << 1) | (((p2 >> bit) & 1u) << 2) |
                                        (((p3 >> bit) & 1u) << 3) | (((p4 >> bit) & 1u) << 4) | (((p5 >> bit) & 1u) << 5) |
                                        (((p6 >> bit) & 1u) << 6);
                    if (dd >= tau[q]) continue;  // tightened by an earlier candidate
                    knn::list_insert<SLOTS>(ld[q], li[q], dd, uint32_t(src_base + bit), lane);
                    tau[q] = knn::list_threshold<SLOTS>(ld[q], k);
                }
            }
        }
        __syncthreads();  // every warp is done with this stage
        if (threadIdx.x == 0 && t + 2 < tiles) {
            knn::mbar_expect_tx(&full_bar[st], TILE_BYTES);
            knn::bulk_g2s(st == 0 ? stage0 : stage1, sliced + (t + 2) * (TILE_BYTES / 4), TILE_BYTES, &full_bar[st]);
        }
    }
    if (lost) {
        if (threadIdx.x == 0) {
            atomicExch(status, kStatusWaitTimeout);
            knn::drain_after_loss(full_bar, lost_tile, tiles);
        }
        return;
    }
#pragma unroll
    for (int q = 0; q < kSlQ; ++q) {
        const uint64_t row = first_row + q;
        if (row >= row_end) continue;
        knn::list_write<SLOTS>(ld[q], li[q], row, k, nbrs + (row - row_begin) * uint64_t(k),
                               dists ? dists + (row - row_begin) * uint64_t(k) : nullptr, lane);
    }
}

// ---- sign-bit codes of any width, with or without residual weighting -----------------------------------
// One plane per component (binary-code mode), K = 8 * nblk <= 120 components.  The first 8 * nblk_p
// components are primary bits: the distance is (h_primary << shift) + h_residual
// (include/cphnsw/core/types.hpp:284-302); nblk_p = 0 is the plain count.  Same list machinery as
// knn_sliced_kernel; the counts are kept as seven planes each and added in bit-sliced form.
constexpr int kWPlanes = 11;  // (120 << 4) + 120 < 2048

template <int SLOTS>
__global__ void __launch_bounds__(kSlWarps * 32)
knn_sliced_binary_kernel(const uint32_t* __restrict__ sliced, const uint8_t* __restrict__ codes, uint64_t n, uint32_t k,
                         uint64_t row_begin, uint64_t row_end, uint32_t* __restrict__ nbrs, uint16_t* __restrict__ dists,
                         uint32_t* __restrict__ status, uint32_t first_wait_polls, int nblk, int nblk_p, int shift) {
    const int K = nblk * 8, CHUNKS = nblk * 2;
    const uint32_t TILE_BYTES = uint32_t(CHUNKS) * 32 * 16;
    extern __shared__ __align__(128) unsigned char sl_smem[];
    uint4* stage0 = reinterpret_cast<uint4*>(sl_smem);
    uint4* stage1 = stage0 + CHUNKS * 32;
    uint4* masks = stage1 + CHUNKS * 32;  // [warp][q][chunk]
    __shared__ uint64_t full_bar[2];
    __shared__ int abort_flag;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t tiles = (n + knn::kTile - 1) / knn::kTile;
    if (threadIdx.x == 0) {
        knn::mbar_init(&full_bar[0], 1);
        knn::mbar_init(&full_bar[1], 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint64_t t = 0; t < 2 && t < tiles; ++t) {
            knn::mbar_expect_tx(&full_bar[t], TILE_BYTES);
            knn::bulk_g2s(t == 0 ? stage0 : stage1, sliced + t * (TILE_BYTES / 4), TILE_BYTES, &full_bar[t]);
        }
    }
    const uint64_t first_row = row_begin + (uint64_t(blockIdx.x) * kSlWarps + warp) * kSlQ;
    uint4* my_masks = masks + size_t(warp) * kSlQ * CHUNKS;
    for (int q = 0; q < kSlQ; ++q) {
        const uint64_t row = min(first_row + q, row_end - 1);
        uint32_t* mw = reinterpret_cast<uint32_t*>(my_masks + q * CHUNKS);
        for (int w = lane; w < K; w += 32) mw[w] = (codes[row * K + w] & 1u) ? kFull : 0u;
    }
    __syncwarp();

    uint32_t ld[kSlQ][SLOTS], li[kSlQ][SLOTS], tau[kSlQ];
#pragma unroll
    for (int q = 0; q < kSlQ; ++q) {
        tau[q] = kFull;
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) ld[q][s] = kFull, li[q][s] = kInvalidNode;
    }

    bool lost = false;
    uint64_t lost_tile = 0;
    for (uint64_t t = 0; t < tiles; ++t) {
        const int st = int(t & 1);
        const uint32_t parity = uint32_t((t >> 1) & 1);
        if (!knn::mbar_wait_bounded(&full_bar[st], parity, t == 0 ? first_wait_polls : knn::kWaitLimit)) abort_flag = 1;
        __syncthreads();
        if (abort_flag) {
            lost = true;
            lost_tile = t;
            break;
        }
        const uint4* tile = st == 0 ? stage0 : stage1;
        const uint64_t group_base = t * knn::kTile + uint64_t(lane) * 32;
        const uint32_t valid = group_base >= n ? 0u : (n - group_base >= 32 ? kFull : ((1u << (n - group_base)) - 1u));

        // S: count planes of the part being summed (weights 1, 2, .., 64); P: those of the primary part
        uint32_t S[kSlQ][7], P[kSlQ][7];
#pragma unroll
        for (int q = 0; q < kSlQ; ++q)
#pragma unroll
            for (int b = 0; b < 7; ++b) S[q][b] = P[q][b] = 0;

#pragma unroll 1
        for (int blk = 0; blk < nblk; ++blk) {
            if (blk == nblk_p) {  // the primary part ends here (nblk_p = 0: there is none)
#pragma unroll
                for (int q = 0; q < kSlQ; ++q)
#pragma unroll
                    for (int b = 0; b < 7; ++b) P[q][b] = S[q][b], S[q][b] = 0;
            }
            const uint4 sa = tile[size_t(blk * 2) * 32 + lane], sb = tile[size_t(blk * 2 + 1) * 32 + lane];
#pragma unroll
            for (int q = 0; q < kSlQ; ++q) {
                const uint4 ma = my_masks[q * CHUNKS + blk * 2], mb = my_masks[q * CHUNKS + blk * 2 + 1];
                // "differs" planes of the block's 8 components, carry-save added into the running count
                uint32_t twosA, twosB, foursA, foursB, e8;
                csa(twosA, S[q][0], S[q][0], sa.x ^ ma.x, sa.y ^ ma.y);
                csa(twosB, S[q][0], S[q][0], sa.z ^ ma.z, sa.w ^ ma.w);
                csa(foursA, S[q][1], S[q][1], twosA, twosB);
                csa(twosA, S[q][0], S[q][0], sb.x ^ mb.x, sb.y ^ mb.y);
                csa(twosB, S[q][0], S[q][0], sb.z ^ mb.z, sb.w ^ mb.w);
                csa(foursB, S[q][1], S[q][1], twosA, twosB);
                csa(e8, S[q][2], S[q][2], foursA, foursB);
                // the weight-8 carry ripples into the 8 / 16 / 32 / 64 planes
                const uint32_t c16 = S[q][3] & e8;
                S[q][3] ^= e8;
                const uint32_t c32 = S[q][4] & c16;
                S[q][4] ^= c16;
                const uint32_t c64 = S[q][5] & c32;
                S[q][5] ^= c32;
                S[q][6] ^= c64;
            }
        }

#pragma unroll
        for (int q = 0; q < kSlQ; ++q) {
            // D = (P << shift) + S, bit-sliced
            uint32_t D[kWPlanes];
#pragma unroll
            for (int b = 0; b < kWPlanes; ++b) D[b] = b < 7 ? P[q][b] : 0u;
#pragma unroll 1
            for (int s = 0; s < shift; ++s) {
#pragma unroll
                for (int b = kWPlanes - 1; b >= 1; --b) D[b] = D[b - 1];
                D[0] = 0;
            }
            uint32_t carry = 0;
#pragma unroll
            for (int b = 0; b < kWPlanes; ++b) {
                const uint32_t r = b < 7 ? S[q][b] : 0u;
                const uint32_t u = D[b] ^ r;
                const uint32_t sum = u ^ carry;
                carry = (D[b] & r) | (u & carry);
                D[b] = sum;
            }
            // candidates with distance < tau[q]
            uint32_t pass;
            if (tau[q] >= (1u << kWPlanes)) {
                pass = kFull;
            } else {
                uint32_t lt = 0, eq = kFull;
#pragma unroll
                for (int b = kWPlanes - 1; b >= 0; --b) {
                    if ((tau[q] >> b) & 1u) {
                        lt |= eq & ~D[b];
                        eq &= D[b];
                    } else {
                        eq &= ~D[b];
                    }
                }
                pass = lt;
            }
            pass &= valid;
            uint32_t lanes = __ballot_sync(kFull, pass != 0);
            while (lanes) {
                const int src = __ffs(lanes) - 1;
                lanes &= lanes - 1;
                uint32_t pm = __shfl_sync(kFull, pass, src);
                uint32_t pl[kWPlanes];
#pragma unroll
                for (int b = 0; b < kWPlanes; ++b) pl[b] = __shfl_sync(kFull, D[b], src);
                const uint64_t src_base = t * knn::kTile + uint64_t(src) * 32;
                while (pm) {
                    const int bit = __ffs(pm) - 1;
                    pm &= pm - 1;
                    uint32_t dd = 0;
#pragma unroll
                    for (int b = 0; b < kWPlanes; ++b) dd |= ((pl[b] >> bit) & 1u) << b;
                    if (dd >= tau[q]) continue;  // tightened by an earlier candidate
                    knn::list_insert<SLOTS>(ld[q], li[q], dd, uint32_t(src_base + bit), lane);
                    tau[q] = knn::list_threshold<SLOTS>(ld[q], k);
                }
            }
        }
        __syncthreads();  // every warp is done with this stage
        if (threadIdx.x == 0 && t + 2 < tiles) {
            knn::mbar_expect_tx(&full_bar[st], TILE_BYTES);
            knn::bulk_g2s(st == 0 ? stage0 : stage1, sliced + (t + 2) * (TILE_BYTES / 4), TILE_BYTES, &full_bar[st]);
        }
    }
    if (lost) {
        if (threadIdx.x == 0) {
            atomicExch(status, kStatusWaitTimeout);
            knn::drain_after_loss(full_bar, lost_tile, tiles);
        }
        return;
    }
#pragma unroll
    for (int q = 0; q < kSlQ; ++q) {
        const uint64_t row = first_row + q;
        if (row >= row_end) continue;
        knn::list_write<SLOTS>(ld[q], li[q], row, k, nbrs + (row - row_begin) * uint64_t(k),
                               dists ? dists + (row - row_begin) * uint64_t(k) : nullptr, lane);
    }
}

template <int SLOTS>
int launch_sliced_binary_t(cphnsw_b200_index* h, const uint32_t* sliced, const uint8_t* codes, uint64_t n, uint32_t k,
                           uint64_t rb, uint64_t re, uint32_t* nbrs, uint16_t* dist, cudaStream_t st) {
    const int nblk = int(h->K / 8), chunks = nblk * 2;
    const int nblk_p = h->residual_bits ? int((h->K - h->residual_bits) / 8) : 0;
    const size_t smem = size_t(2) * chunks * 32 * 16 + size_t(kSlWarps) * kSlQ * chunks * 16;
    auto kernel = knn_sliced_binary_kernel<SLOTS>;
    CPB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    const uint64_t blocks = (re - rb + kSlWarps * kSlQ - 1) / (kSlWarps * kSlQ);
    LaunchTimer timer(h, kKernelKnn, st);
    kernel<<<unsigned(blocks), kSlWarps * 32, smem, st>>>(sliced, codes, n, k, rb, re, nbrs, dist, h->d_status.as<uint32_t>(), h->first_wait_polls, nblk,
                                                         nblk_p, int(h->residual_bits ? h->residual_shift : 0));
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

template <typename CompT, int NB, int NBLK, int SLOTS, int WARPS>
int launch_sliced_t(cphnsw_b200_index* h, const uint32_t* sliced, const CompT* codes, uint64_t n, uint32_t k,
                    uint64_t rb, uint64_t re, uint32_t* nbrs, uint16_t* dist, cudaStream_t st) {
    constexpr int CHUNKS = NBLK * 8 * NB / 4;
    const size_t smem = size_t(2) * CHUNKS * 32 * 16 + size_t(WARPS) * kSlQ * CHUNKS * 16;
    auto kernel = knn_sliced_kernel<CompT, NB, NBLK, SLOTS, WARPS>;
    CPB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    const uint64_t rows = re - rb;
    const uint64_t blocks = (rows + WARPS * kSlQ - 1) / (WARPS * kSlQ);
    LaunchTimer timer(h, kKernelKnn, st);
    kernel<<<unsigned(blocks), WARPS * 32, smem, st>>>(sliced, codes, n, k, rb, re, nbrs, dist, h->d_status.as<uint32_t>(), h->first_wait_polls);
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

template <typename CompT, int NB, int NBLK, int WARPS>
int launch_sliced_slots(cphnsw_b200_index* h, const uint32_t* sliced, const CompT* codes, uint64_t n, uint32_t k,
                        uint64_t rb, uint64_t re, uint32_t* nbrs, uint16_t* dist, cudaStream_t st) {
    const uint32_t need = k + 1;
    if (need <= 64) return launch_sliced_t<CompT, NB, NBLK, 2, WARPS>(h, sliced, codes, n, k, rb, re, nbrs, dist, st);
    if (need <= 96) return launch_sliced_t<CompT, NB, NBLK, 3, WARPS>(h, sliced, codes, n, k, rb, re, nbrs, dist, st);
    return launch_sliced_t<CompT, NB, NBLK, 4, WARPS>(h, sliced, codes, n, k, rb, re, nbrs, dist, st);
}

}  // namespace

// Sign-bit codes that take knn_sliced_binary_kernel: one-byte components, whole blocks of 8 components
// in the code and in its primary part, at most 120 components.
static bool knn_sliced_binary_general(const cphnsw_b200_index* h) {
    if (h->K % 8 != 0 || h->K > 120) return false;
    if (h->residual_bits) return (h->K - h->residual_bits) % 8 == 0;
    return h->K != 16 && h->K != 32 && h->K != 64;  // those widths have their own instantiations
}

// Planes per component: 8 for uint8 codes, 11 for uint16 codes of padded dim 1024 (10 index bits +
// sign), 1 in binary-code mode (a component is its sign bit).  K = 16, 32 or 64 (64: not with 11 planes).
bool knn_sliced_supported(const cphnsw_b200_index* h) {
    if (h->binary_codes && h->comp_bytes == 1 && knn_sliced_binary_general(h)) return true;
    if (h->residual_bits) return false;  // weighted (combined) distance of wider components: the byte-wise kernel
    if (h->K != 16 && h->K != 32 && h->K != 64) return false;
    if (h->binary_codes) return true;
    if (h->comp_bytes == 1) return true;
    return h->comp_bytes == 2 && h->P == 1024 && h->K != 64;
}

namespace {
template <typename CompT, int NB, int WARPS>
int launch_sliced_k(cphnsw_b200_index* h, const uint32_t* sl, const CompT* codes, uint64_t n, uint32_t k, uint64_t rb,
                    uint64_t re, uint32_t* nbrs, uint16_t* dist, cudaStream_t st) {
    if (h->K == 16) return launch_sliced_slots<CompT, NB, 2, WARPS>(h, sl, codes, n, k, rb, re, nbrs, dist, st);
    if (h->K == 32) return launch_sliced_slots<CompT, NB, 4, WARPS>(h, sl, codes, n, k, rb, re, nbrs, dist, st);
    if constexpr (NB <= 8) return launch_sliced_slots<CompT, NB, 8, WARPS>(h, sl, codes, n, k, rb, re, nbrs, dist, st);
    set_error("bit-sliced kNN: K = 64 is not available with 11-plane components");
    return CPHNSW_B200_E_UNSUPPORTED;
}
}  // namespace

int launch_knn_graph_sliced(cphnsw_b200_index* h, const void* d_codes, uint64_t n, uint32_t k, uint64_t row_begin,
                            uint64_t row_end, uint32_t* d_nbrs, uint16_t* d_dist, cudaStream_t st) {
    const int K = int(h->K);
    const bool u16 = h->comp_bytes == 2;
    const int NB = h->binary_codes ? 1 : (u16 ? 11 : 8);
    const uint64_t tiles = (n + knn::kTile - 1) / knn::kTile;
    const uint64_t n_groups = tiles * 32;
    const size_t sliced_bytes = size_t(tiles) * K * NB * 32 * 4;
    CPB_TRY(h->s_sliced.reserve(sliced_bytes + 16));
    {
        const uint64_t threads = n_groups * 32;
        const unsigned grid = unsigned((threads + 255) / 256);
        if (u16)
            slice_codes_kernel<uint16_t><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(d_codes), n, K, NB,
                                                               h->s_sliced.as<uint32_t>(), n_groups);
        else
            slice_codes_kernel<uint8_t><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(d_codes), n, K, NB,
                                                              h->s_sliced.as<uint32_t>(), n_groups);
        h->launches++;
        CPB_CUDA(cudaGetLastError());
    }
    const uint32_t* sl = h->s_sliced.as<uint32_t>();
    if (u16) {
        const uint16_t* codes = static_cast<const uint16_t*>(d_codes);
        if (NB == 1) return launch_sliced_k<uint16_t, 1, kSlWarps>(h, sl, codes, n, k, row_begin, row_end, d_nbrs, d_dist, st);
        return launch_sliced_k<uint16_t, 11, 8>(h, sl, codes, n, k, row_begin, row_end, d_nbrs, d_dist, st);
    }
    const uint8_t* codes = static_cast<const uint8_t*>(d_codes);
    if (NB == 1 && knn_sliced_binary_general(h)) {
        const uint32_t need = k + 1;
        if (need <= 64) return launch_sliced_binary_t<2>(h, sl, codes, n, k, row_begin, row_end, d_nbrs, d_dist, st);
        if (need <= 96) return launch_sliced_binary_t<3>(h, sl, codes, n, k, row_begin, row_end, d_nbrs, d_dist, st);
        return launch_sliced_binary_t<4>(h, sl, codes, n, k, row_begin, row_end, d_nbrs, d_dist, st);
    }
    if (NB == 1) return launch_sliced_k<uint8_t, 1, kSlWarps>(h, sl, codes, n, k, row_begin, row_end, d_nbrs, d_dist, st);
    return launch_sliced_k<uint8_t, 8, kSlWarps>(h, sl, codes, n, k, row_begin, row_end, d_nbrs, d_dist, st);
}

}  // namespace cpb
