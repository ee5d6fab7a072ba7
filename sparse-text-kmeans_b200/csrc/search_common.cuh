// Pieces shared by the search kernels: launch arguments, the (distance, id) order, the two metrics
// (asymmetric CP score in its fixed tree order, symmetric code distance) and the shared-memory
// bitonic sort.  See search.cu for the algorithm.
#pragma once

#include <cmath>

#include "common.cuh"

namespace cpb {
namespace srch {

constexpr uint32_t kFull = 0xffffffffu;
constexpr uint32_t kExpanded = 0x80000000u; // top bit of a stored id: the member has been expanded
constexpr uint32_t kIdMask = 0x7fffffffu;
constexpr int kCoopMax = 8;                 // up to this many fresh nodes are scored by the whole warp

struct SearchArgs {
    const float* tables;   // [nq][K][P] (asymmetric metric)
    const void* qcodes;    // [nq][K] query codes (symmetric metric)
    const float* queries;  // [nq][dim] (rerank only)
    const void* codes;     // [n][K] components
    const uint32_t* packed;  // binary-code mode: [n][packed_words] sign bits, 32 per word (else nullptr)
    int packed_words;
    const uint32_t* adj;   // [n][M]
    const float* vectors;  // [n][dim] (rerank only)
    const uint32_t* entry;     // ids scored for every query before the walk
    const void* entry_codes;   // their codes, gathered contiguously [n_entry][K]
    uint32_t n_entry, n_seed;  // the n_seed best of the scan seed the walk
    uint64_t n;
    uint32_t nq;
    int K, P, dim, M, comp_bytes;
    uint32_t qsm_floats;              // size of the per-warp query area: the query vector, then (symmetric metric) the query code
    uint32_t qvec_floats;             // its first part: the query vector padded to a multiple of 4 floats
    uint32_t per_warp_smem;           // bytes of shared memory per warp (multiple of 16)
    uint32_t beam, cap, k, rerank_k;  // cap: power of two >= max(32, beam, n_seed), the size of W's arrays
    uint8_t* visited;    // [warp slots][vis_stride]: epoch of the last query that visited the node
    uint64_t vis_stride; // bytes per warp slot (n rounded up to 16)
    uint32_t* epochs;    // [warp slots]: last epoch used by the slot (persists across launches)
    uint32_t* out_ids;
    float* out_dist;
    uint32_t* stats;
    uint32_t* next_query;  // work counter, zero at launch
    int rows_distinct;     // no adjacency row lists a node twice (checked when the adjacency is set)
    int table_in_smem;     // two-warp kernel: the query table is copied to shared memory (else read from global memory)
    int resid_kp;          // residual codes: the first resid_kp components are primary and count 1 + resid_mul
    int resid_mul;         //   in the symmetric distance (0: plain count)
    int scan_only;         // brute_force_search: score all n nodes (entry == nullptr: ids 0..n-1), keep the n_seed best, no walk
};

__device__ __forceinline__ void prefetch_l1(const void* p) {
    asm volatile("prefetch.global.L1 [%0];" ::"l"(p));
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

__device__ __forceinline__ bool key_less(float da, uint32_t ia, float db, uint32_t ib) {
    return da < db || (da == db && ia < ib);
}

template <bool U16>
__device__ __forceinline__ uint32_t load_component(const unsigned char* row, int r) {
    return U16 ? uint32_t(reinterpret_cast<const uint16_t*>(row)[r]) : uint32_t(row[r]);
}

// signed table value of rotation r for component `comp` (+0 for r >= K)
__device__ __forceinline__ float signed_term(const float* table, int r, int K, int P, uint32_t comp) {
    if (r >= K) return 0.0f;
    const float val = table[r * P + int(comp >> 1)];
    return (comp & 1u) ? -val : val;
}

// One lane scores one node: the 32 terms of each block are combined in the balanced-tree order
// (j with j+16, then +8, +4, +2, +1), blocks are added in sequence.
template <bool U16>
__device__ __forceinline__ float asym_distance_lane(const float* table, const void* codes, uint32_t row_index,
                                                    int K, int P) {
    const int row_bytes = K * (U16 ? 2 : 1);
    const unsigned char* row = static_cast<const unsigned char*>(codes) + size_t(row_index) * row_bytes;
    const bool vec = (row_bytes & 15) == 0;
    float acc = 0.0f;
    for (int c0 = 0; c0 < K; c0 += 32) {
        float t[32];
        if (vec) {
            constexpr int kPerWord = U16 ? 2 : 4;           // components per 32-bit word
            constexpr int kWords = 32 / kPerWord;           // words per block of 32 components
            const uint4* r4 = reinterpret_cast<const uint4*>(row + size_t(c0) * (U16 ? 2 : 1));
            uint32_t w[kWords];
#pragma unroll
            for (int i = 0; i < kWords / 4; ++i) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (c0 + i * 4 * kPerWord < K) v = __ldg(r4 + i);
                w[4 * i] = v.x, w[4 * i + 1] = v.y, w[4 * i + 2] = v.z, w[4 * i + 3] = v.w;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const uint32_t word = w[j / kPerWord];
                const uint32_t comp = U16 ? ((word >> (16 * (j % 2))) & 0xffffu) : ((word >> (8 * (j % 4))) & 0xffu);
                t[j] = signed_term(table, c0 + j, K, P, comp);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int r = c0 + j;
                t[j] = signed_term(table, r, K, P, r < K ? load_component<U16>(row, r) : 0u);
            }
        }
#pragma unroll
        for (int step = 16; step >= 1; step >>= 1) {
#pragma unroll
            for (int j = 0; j < step; ++j) t[j] = __fadd_rn(t[j], t[j + step]);
        }
        acc = __fadd_rn(acc, t[0]);
    }
    return -acc;
}

// Symmetric metric (search_multiprobe): number of components in which the node's code differs
// from the query code staged in shared memory, as a float.
template <bool U16>
__device__ __forceinline__ float sym_distance_lane(const unsigned char* qcode, const void* codes, uint32_t row_index,
                                                   int K, int kp = 0, int mul = 0) {
    const int row_bytes = K * (U16 ? 2 : 1);
    const unsigned char* row = static_cast<const unsigned char*>(codes) + size_t(row_index) * row_bytes;
    uint32_t d = 0;
    if ((row_bytes & 3) == 0) {
        constexpr uint32_t LO = U16 ? 0x7fff7fffu : 0x7f7f7f7fu;
        const uint32_t* r32 = reinterpret_cast<const uint32_t*>(row);
        const uint32_t* q32 = reinterpret_cast<const uint32_t*>(qcode);
        if (!mul) {
            for (int w = 0; w < row_bytes / 4; ++w) {
                const uint32_t x = q32[w] ^ __ldg(r32 + w);
                d += __popc((((x & LO) + LO) | x) & ~LO);  // one flag per differing byte / halfword
            }
        } else {  // residual codes: a primary word counts 1 + mul (kp * component size is a multiple of 4)
            const int wp = kp * (U16 ? 2 : 1) / 4;
            for (int w = 0; w < row_bytes / 4; ++w) {
                const uint32_t x = q32[w] ^ __ldg(r32 + w);
                const uint32_t c = __popc((((x & LO) + LO) | x) & ~LO);
                d += w < wp ? c * uint32_t(1 + mul) : c;
            }
        }
    } else {
        for (int r = 0; r < K; ++r)
            d += (load_component<U16>(row, r) != load_component<U16>(qcode, r)) ? (r < kp ? 1 + mul : 1) : 0;
    }
    return float(d);
}

// The same distance on sign bits packed 32 per word (binary-code mode): the Hamming distance is the popcount of the
// XOR; with residual codes the first kp bits are primary and count 1 + mul.  q holds the query's packed code.
__device__ __forceinline__ float packed_distance_lane(const uint32_t* q, const uint32_t* packed, uint32_t row_index, int words,
                                                      int kp, int mul) {
    const uint32_t* x = packed + size_t(row_index) * words;
    uint32_t d = 0;
    for (int w = 0; w < words; ++w) {
        const uint32_t v = q[w] ^ __ldg(x + w);
        d += __popc(v);
        if (mul) {
            const int lo = kp - 32 * w;  // primary bits in this word
            const uint32_t pm = lo >= 32 ? 0xffffffffu : (lo > 0 ? (1u << lo) - 1u : 0u);
            d += uint32_t(mul) * __popc(v & pm);
        }
    }
    return float(d);
}

// The whole warp scores one node: lane j owns rotation c0 + j of each block; the butterfly
// reduction adds exactly the pairs the one-lane form adds.  `comp` is this lane's component of
// block 0 (K <= 32 here; asym_distance_coop2 takes 32 < K <= 64).
__device__ __forceinline__ float asym_distance_coop(const float* table, int K, int P, uint32_t comp, int lane) {
    float t = signed_term(table, lane, K, P, comp);
#pragma unroll
    for (int step = 16; step >= 1; step >>= 1) t = __fadd_rn(t, __shfl_xor_sync(kFull, t, step));
    return -__fadd_rn(0.0f, t);
}

// The same for two blocks (32 < K <= 64): lane j owns rotations j and 32 + j; the block sums are formed side by
// side and added in block order, as the one-lane form does.
__device__ __forceinline__ float asym_distance_coop2(const float* table, int K, int P, uint32_t comp_lo, uint32_t comp_hi,
                                                     int lane) {
    float t0 = signed_term(table, lane, K, P, comp_lo);
    float t1 = signed_term(table, 32 + lane, K, P, comp_hi);
#pragma unroll
    for (int step = 16; step >= 1; step >>= 1) {
        t0 = __fadd_rn(t0, __shfl_xor_sync(kFull, t0, step));
        t1 = __fadd_rn(t1, __shfl_xor_sync(kFull, t1, step));
    }
    return -__fadd_rn(__fadd_rn(0.0f, t0), t1);
}

// ---- warp-wide bitonic sort of n (a power of two) (distance, id) pairs in shared memory ------------
// ascending by (distance, id); runtime loops keep the code small, each lane handles n/64 pairs
// per stage.
__device__ __forceinline__ void warp_sort_smem(float* d, uint32_t* id, int n, int lane) {
    for (int k2 = 2; k2 <= n; k2 <<= 1) {
        for (int j = k2 >> 1; j > 0; j >>= 1) {
            for (int t = lane; t < n / 2; t += 32) {
                const int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));  // index with bit j clear
                const int hi = lo | j;
                const bool asc = (lo & k2) == 0;
                const float dl = d[lo], dh = d[hi];
                const uint32_t il = id[lo], ih = id[hi];
                const bool hi_less = key_less(dh, ih, dl, il);
                if (hi_less == asc) {
                    d[lo] = dh;
                    id[lo] = ih;
                    d[hi] = dl;
                    id[hi] = il;
                }
            }
            __syncwarp();
        }
    }
}

// The k smallest of n pairs, ascending, into positions [0, k): k rounds of "find the smallest of [r, n), swap it to r".
// For the few results a query returns this is a fraction of the full sort (k = 10 of 500 reranked candidates: about
// 1,500 instead of 7,000 warp instructions) and yields the same pairs in the same order, the order being total.
constexpr uint32_t kSelectMax = 16;  // above this many results the full sort is taken
__device__ __forceinline__ void warp_select_smem(float* d, uint32_t* id, int n, int k, int lane) {
    for (int r = 0; r < k && r < n; ++r) {
        float bd = INFINITY;
        uint32_t bi = kInvalidNode;
        int bp = r;
        for (int p = r + lane; p < n; p += 32) {
            const float v = d[p];
            const uint32_t w = id[p];
            if (key_less(v, w, bd, bi)) {
                bd = v;
                bi = w;
                bp = p;
            }
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const float od = __shfl_xor_sync(kFull, bd, o);
            const uint32_t oi = __shfl_xor_sync(kFull, bi, o);
            const int op = __shfl_xor_sync(kFull, bp, o);
            if (key_less(od, oi, bd, bi)) {
                bd = od;
                bi = oi;
                bp = op;
            }
        }
        if (lane == 0 && bi != kInvalidNode && bp != r) {
            const float td = d[r];
            const uint32_t ti = id[r];
            d[r] = bd;
            id[r] = bi;
            d[bp] = td;
            id[bp] = ti;
        }
        __syncwarp();
    }
}

// bitonic sort of n (a power of two) pairs by (distance, id without the expanded flag); the flag travels with the id
__device__ __forceinline__ void warp_sort_flagged(float* d, uint32_t* id, int n, int lane) {
    for (int k2 = 2; k2 <= n; k2 <<= 1) {
        for (int j = k2 >> 1; j > 0; j >>= 1) {
            for (int t = lane; t < n / 2; t += 32) {
                const int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                const int hi = lo | j;
                const bool asc = (lo & k2) == 0;
                const float dl = d[lo], dh = d[hi];
                const uint32_t il = id[lo], ih = id[hi];
                const bool hi_less = key_less(dh, ih & kIdMask, dl, il & kIdMask);
                if (hi_less == asc) {
                    d[lo] = dh;
                    id[lo] = ih;
                    d[hi] = dl;
                    id[hi] = il;
                }
            }
            __syncwarp();
        }
    }
}

}  // namespace srch
}  // namespace cpb
