// Pieces shared by the two kNN-graph kernels (byte-wise and bit-sliced distance): bounded
// mbarrier waits, 1-D bulk asynchronous copies, and the running best-(k+1) list of a query row
// that a warp keeps sorted across its registers.
#pragma once

#include "common.cuh"

namespace cpb {
namespace knn {

constexpr uint32_t kFull = 0xffffffffu;
constexpr int kTile = 1024;               // candidates per shared-memory stage
constexpr uint32_t kWaitLimit = 1u << 22;  // polls before a wait is declared lost

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll may itself suspend for a short,
// hardware-bounded time) and reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// After a wait for tile t was lost: the copies that can still be in flight are those of tiles t and
// t + 1 (tile u lands in stage u & 1 and completes that barrier's phase of parity (u >> 1) & 1).
// They get the full poll limit to land before the block and its shared memory go away.
__device__ __forceinline__ void drain_after_loss(uint64_t* full_bar, uint64_t t, uint64_t tiles) {
    for (uint64_t u = t; u < t + 2 && u < tiles; ++u)
        mbar_wait_bounded(&full_bar[u & 1], uint32_t((u >> 1) & 1), kWaitLimit);
}
// 1-D bulk asynchronous copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// The running list of one query row: element of rank (s*32 + lane) sits in slot s of lane
// `lane`, ascending by (distance, id); unused places hold (0xFFFFFFFF, no node).
// list_place puts (dd, id), known to every lane, at rank p (warp-uniform) and moves the elements
// of rank >= p one place down; the last element falls off.
template <int SLOTS>
__device__ __forceinline__ void list_place(uint32_t (&ld)[SLOTS], uint32_t (&li)[SLOTS], int p, uint32_t dd, uint32_t id,
                                           int lane) {
#pragma unroll
    for (int s = SLOTS - 1; s >= 0; --s) {
        uint32_t ud = __shfl_up_sync(kFull, ld[s], 1);
        uint32_t ui = __shfl_up_sync(kFull, li[s], 1);
        if (s > 0) {
            uint32_t cd = __shfl_sync(kFull, ld[s - 1], 31);
            uint32_t ci = __shfl_sync(kFull, li[s - 1], 31);
            if (lane == 0) {
                ud = cd;
                ui = ci;
            }
        }
        const int rank = s * 32 + lane;
        if (rank > p) {
            ld[s] = ud;
            li[s] = ui;
        } else if (rank == p) {
            ld[s] = dd;
            li[s] = id;
        }
    }
}

// Inserts (dd, id) where id is larger than every id already kept (rows are swept in ascending
// candidate order): its rank is the number of kept elements with distance <= dd.
template <int SLOTS>
__device__ __forceinline__ void list_insert(uint32_t (&ld)[SLOTS], uint32_t (&li)[SLOTS], uint32_t dd, uint32_t id,
                                            int lane) {
    int p = 0;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) p += __popc(__ballot_sync(kFull, ld[s] <= dd));
    list_place<SLOTS>(ld, li, p, dd, id, lane);
}

// The same for ids in any order: the rank is the number of kept elements below (dd, id).
template <int SLOTS>
__device__ __forceinline__ int list_rank_keyed(const uint32_t (&ld)[SLOTS], const uint32_t (&li)[SLOTS], uint32_t dd,
                                               uint32_t id) {
    int p = 0;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) p += __popc(__ballot_sync(kFull, ld[s] < dd || (ld[s] == dd && li[s] < id)));
    return p;
}

// Admission threshold: the distance of the element of rank k (the (k+1)-th: one place is kept
// for the row's own id, which is dropped at write-out).
template <int SLOTS>
__device__ __forceinline__ uint32_t list_threshold(const uint32_t (&ld)[SLOTS], uint32_t k) {
    uint32_t tk = kFull;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const uint32_t v = __shfl_sync(kFull, ld[s], int(k & 31));
        if (s == int(k >> 5)) tk = v;
    }
    return tk;
}

// Writes one finished row: the k best other than the row itself, padded with 0xFFFFFFFF / 0xFFFF.
template <int SLOTS>
__device__ __forceinline__ void list_write(const uint32_t (&ld)[SLOTS], const uint32_t (&li)[SLOTS], uint64_t row,
                                           uint32_t k, uint32_t* out_n, uint16_t* out_d, int lane) {
    int selfrank = 0x7fffffff, valid = 0;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        uint32_t ms = __ballot_sync(kFull, li[s] == uint32_t(row));
        if (ms && selfrank == 0x7fffffff) selfrank = s * 32 + __ffs(ms) - 1;
        valid += __popc(__ballot_sync(kFull, li[s] != kInvalidNode));
    }
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const int rank = s * 32 + lane;
        if (li[s] == kInvalidNode || rank == selfrank) continue;
        const int o = rank - (rank > selfrank ? 1 : 0);
        if (o < int(k)) {
            out_n[o] = li[s];
            if (out_d) out_d[o] = uint16_t(ld[s]);
        }
    }
    const int n_out = valid - (selfrank != 0x7fffffff ? 1 : 0);
    for (int o = n_out + lane; o < int(k); o += 32) {
        out_n[o] = kInvalidNode;
        if (out_d) out_d[o] = 0xFFFF;
    }
}

}  // namespace knn
}  // namespace cpb
