// search_multiprobe support: the multiprobe sequence of a query's cross-polytope code, and the
// merge of the per-probe result lists.
//
// Probe sequence (resources/cross-polytope-lsh/consolidated.tex:391-425; the data CPQuery keeps for
// it, include/cphnsw/core/types.hpp:332-336): per rotation the coordinates of the rotated query are
// ranked by (|x| descending, index ascending); taking the coordinate of rank v instead of the
// winner costs (|x|_(0) - |x|_(v))^2; a probe picks one rank per rotation and is scored by the sum
// of its costs over rotations in ascending rotation order (fp32, one rounding per add).  Probes
// come out in ascending (score, creation number) order, the primary code first: after a probe whose
// last modified rotation is j, its successors are "raise the rank of rotation j by one" and "set
// rotation j' to rank 1" for every j' > j, created in that order, so every rank combination has
// exactly one derivation and the order is reproducible.
//
// One warp per query; the per-rotation ranking, the successor scores and the pool scan are spread
// over the lanes.
#include <cmath>

#include "common.cuh"

namespace cpb {
namespace {

constexpr uint32_t kFull = 0xffffffffu;
constexpr uint32_t kNoParent = 0xffffffffu;

struct ProbeArgs {
    const float* rotated;  // [nq][K][P]
    uint32_t nq;
    int K, P, T, V;        // V = min(P, T + 1) ranks a probe can use
    int pool_cap;          // K + (T - 1) * (K + 1)
    void* out;             // [nq][T][K] components
};

template <bool U16>
__global__ void probe_codes_kernel(ProbeArgs a) {
    extern __shared__ __align__(16) unsigned char pr_smem[];
    const int lane = threadIdx.x & 31;
    const int K = a.K, P = a.P, T = a.T, V = a.V;
    // per-block (one warp) shared arrays
    float* cost = reinterpret_cast<float*>(pr_smem);                  // [K][V]
    uint32_t* idx = reinterpret_cast<uint32_t*>(cost + K * V);        // [K][V]
    float* pscore = reinterpret_cast<float*>(idx + K * V);            // [pool_cap]
    uint32_t* pparent = reinterpret_cast<uint32_t*>(pscore + a.pool_cap);
    uint16_t* prot = reinterpret_cast<uint16_t*>(pparent + a.pool_cap);
    uint16_t* prank = prot + a.pool_cap;
    uint16_t* last = prank + a.pool_cap;                              // [T]
    uint8_t* ranks = reinterpret_cast<uint8_t*>(last + T);            // [T][K]

    for (uint32_t q = blockIdx.x; q < a.nq; q += gridDim.x) {
        // ---- rank the coordinates of every rotation: V rounds of "next in (|x| desc, index asc) order"
        for (int r = 0; r < K; ++r) {
            const float* x = a.rotated + (size_t(q) * K + r) * P;
            float prev_a = INFINITY;  // key of the previous winner: everything after it is still eligible
            int prev_i = -1;
            float top = 0.0f;
            for (int v = 0; v < V; ++v) {
                float ba = -1.0f;
                int bi = 0x7fffffff;
                for (int i = lane; i < P; i += 32) {
                    const float av = fabsf(__ldg(x + i));
                    const bool after_prev = av < prev_a || (av == prev_a && i > prev_i);
                    if (after_prev && (av > ba || (av == ba && i < bi))) {
                        ba = av;
                        bi = i;
                    }
                }
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) {
                    const float oa = __shfl_xor_sync(kFull, ba, o);
                    const int oi = __shfl_xor_sync(kFull, bi, o);
                    if (oa > ba || (oa == ba && oi < bi)) {
                        ba = oa;
                        bi = oi;
                    }
                }
                if (v == 0) top = ba;
                if (lane == 0) {
                    const float d = __fsub_rn(top, ba);
                    cost[r * V + v] = __fmul_rn(d, d);
                    idx[r * V + v] = uint32_t(bi);
                }
                prev_a = ba;
                prev_i = bi;
            }
        }
        __syncwarp();

        // ---- best-first enumeration of rank combinations
        int npool = 0, nprobe = 1;
        for (int r = lane; r < K; r += 32) ranks[r] = 0;
        if (lane == 0) last[0] = 0;
        __syncwarp();
        // children of probe `parent`, created in the fixed order: raise (if any), then j' ascending
        auto push_children = [&](int parent) {
            const bool primary = parent == 0;
            const int j = primary ? 0 : int(last[parent]);
            const uint8_t* rk = ranks + size_t(parent) * K;
            const bool can_raise = !primary && int(rk[j]) + 1 < V;
            const int first_set = primary ? 0 : j + 1;
            const int nset = V >= 2 ? K - first_set : 0;
            const int nchild = (can_raise ? 1 : 0) + nset;
            for (int c = lane; c < nchild; c += 32) {
                int rot, rank;
                if (can_raise && c == 0) {
                    rot = j;
                    rank = int(rk[j]) + 1;
                } else {
                    rot = first_set + c - (can_raise ? 1 : 0);
                    rank = 1;
                }
                float s = 0.0f;
                for (int r = 0; r < K; ++r) {
                    const int rr = r == rot ? rank : int(rk[r]);
                    if (rr) s = __fadd_rn(s, cost[r * V + rr]);
                }
                pscore[npool + c] = s;
                pparent[npool + c] = uint32_t(parent);
                prot[npool + c] = uint16_t(rot);
                prank[npool + c] = uint16_t(rank);
            }
            npool += nchild;
            __syncwarp();
        };
        push_children(0);
        while (nprobe < T) {
            // unused pool item with the smallest (score, creation number)
            float bs = INFINITY;
            int bi = 0x7fffffff;
            for (int i = lane; i < npool; i += 32) {
                if (pparent[i] != kNoParent && (bi == 0x7fffffff || pscore[i] < bs)) {
                    bs = pscore[i];
                    bi = i;
                }
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                const float os = __shfl_xor_sync(kFull, bs, o);
                const int oi = __shfl_xor_sync(kFull, bi, o);
                if (oi != 0x7fffffff && (bi == 0x7fffffff || os < bs || (os == bs && oi < bi))) {
                    bs = os;
                    bi = oi;
                }
            }
            if (bi == 0x7fffffff) break;  // fewer than T distinct probes exist
            const int parent = int(pparent[bi]), rot = int(prot[bi]), rank = int(prank[bi]);
            __syncwarp();
            for (int r = lane; r < K; r += 32)
                ranks[size_t(nprobe) * K + r] = r == rot ? uint8_t(rank) : ranks[size_t(parent) * K + r];
            if (lane == 0) {
                last[nprobe] = uint16_t(rot);
                pparent[bi] = kNoParent;
            }
            __syncwarp();
            push_children(nprobe);
            ++nprobe;
        }

        // ---- probe codes (a short sequence repeats its last probe)
        for (int t = 0; t < T; ++t) {
            const uint8_t* rk = ranks + size_t(min(t, nprobe - 1)) * K;
            for (int r = lane; r < K; r += 32) {
                const uint32_t i = idx[r * V + rk[r]];
                const float val = __ldg(a.rotated + (size_t(q) * K + r) * P + i);
                const uint32_t comp = (i << 1) | (val < 0.0f ? 1u : 0u);
                const size_t o = (size_t(q) * T + t) * K + r;
                if (U16) static_cast<uint16_t*>(a.out)[o] = uint16_t(comp);
                else static_cast<uint8_t*>(a.out)[o] = uint8_t(comp);
            }
        }
        __syncwarp();
    }
}

// ---- merge of per-probe results: per query the union of T lists of k (id, distance), every id
// once with its smallest distance, ascending by (distance, id), best k.  One warp per query.
__device__ __forceinline__ bool key_less(float da, uint32_t ia, float db, uint32_t ib) {
    return da < db || (da == db && ia < ib);
}

__global__ void merge_probes_kernel(const uint32_t* __restrict__ ids, const float* __restrict__ dist, uint32_t nq, int T,
                                    int k, int npad, uint32_t* __restrict__ out_ids, float* __restrict__ out_dist) {
    extern __shared__ __align__(16) unsigned char mg_smem[];
    const int lane = threadIdx.x & 31;
    uint32_t* sid = reinterpret_cast<uint32_t*>(mg_smem);
    float* sd = reinterpret_cast<float*>(sid + npad);
    uint32_t* oid = reinterpret_cast<uint32_t*>(sd + npad);  // [k] ids already emitted
    for (uint32_t q = blockIdx.x; q < nq; q += gridDim.x) {
        const int n = T * k;
        for (int i = lane; i < npad; i += 32) {
            sid[i] = i < n ? ids[size_t(q) * n + i] : kInvalidNode;
            sd[i] = i < n ? dist[size_t(q) * n + i] : INFINITY;
        }
        __syncwarp();
        // bitonic sort ascending by (distance, id); an id's first occurrence then carries its minimum
        for (int k2 = 2; k2 <= npad; k2 <<= 1)
            for (int j = k2 >> 1; j > 0; j >>= 1) {
                for (int t = lane; t < npad / 2; t += 32) {
                    const int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1)), hi = lo | j;
                    const bool asc = (lo & k2) == 0;
                    const float dl = sd[lo], dh = sd[hi];
                    const uint32_t il = sid[lo], ih = sid[hi];
                    if (key_less(dh, ih, dl, il) == asc) {
                        sd[lo] = dh, sid[lo] = ih, sd[hi] = dl, sid[hi] = il;
                    }
                }
                __syncwarp();
            }
        int nout = 0;
        for (int p = 0; p < n && nout < k; ++p) {
            const uint32_t id = sid[p];
            if (id == kInvalidNode) break;  // padding sorts last
            bool dup = false;
            for (int i = lane; i < nout; i += 32) dup |= oid[i] == id;
            if (__any_sync(kFull, dup)) continue;
            if (lane == 0) {
                oid[nout] = id;
                out_ids[size_t(q) * k + nout] = id;
                out_dist[size_t(q) * k + nout] = sd[p];
            }
            ++nout;
            __syncwarp();
        }
        for (int i = nout + lane; i < k; i += 32) {
            out_ids[size_t(q) * k + i] = kInvalidNode;
            out_dist[size_t(q) * k + i] = INFINITY;
        }
        __syncwarp();
    }
}

}  // namespace

int launch_probe_codes(cphnsw_b200_index* h, const float* d_rotated, uint64_t nq, uint32_t T, void* d_out,
                       cudaStream_t st) {
    if (nq == 0) return 0;
    ProbeArgs a;
    a.rotated = d_rotated;
    a.nq = uint32_t(nq);
    a.K = int(h->K);
    a.P = int(h->P);
    a.T = int(T);
    a.V = int(h->P < uint64_t(T) + 1 ? h->P : uint64_t(T) + 1);
    a.pool_cap = a.K + (a.T - 1) * (a.K + 1) + 1;
    a.out = d_out;
    size_t smem = size_t(a.K) * a.V * 8 + size_t(a.pool_cap) * (4 + 4 + 2 + 2) + size_t(a.T) * 2 + size_t(a.T) * a.K;
    smem = (smem + 15) & ~size_t(15);
    if (smem > 200 * 1024) {
        set_error("search_multiprobe: K=%d with %d probes needs %zu bytes of shared memory per query (max 204800)", a.K,
                  a.T, smem);
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    const unsigned grid = unsigned(nq < uint64_t(h->sm_count) * 8 ? nq : uint64_t(h->sm_count) * 8);
    if (h->comp_bytes == 2) {
        CPB_CUDA(allow_max_dynamic_smem(probe_codes_kernel<true>));
        probe_codes_kernel<true><<<grid, 32, smem, st>>>(a);
    } else {
        CPB_CUDA(allow_max_dynamic_smem(probe_codes_kernel<false>));
        probe_codes_kernel<false><<<grid, 32, smem, st>>>(a);
    }
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

int launch_merge_probes(cphnsw_b200_index* h, const uint32_t* d_ids, const float* d_dist, uint64_t nq, uint32_t T,
                        uint32_t k, uint32_t* d_out_ids, float* d_out_dist, cudaStream_t st) {
    if (nq == 0) return 0;
    int npad = 32;
    while (npad < int(T * k)) npad <<= 1;
    const size_t smem = size_t(npad) * 8 + size_t(k) * 4;
    CPB_CUDA(allow_max_dynamic_smem(merge_probes_kernel));
    const unsigned grid = unsigned(nq < uint64_t(h->sm_count) * 8 ? nq : uint64_t(h->sm_count) * 8);
    merge_probes_kernel<<<grid, 32, smem, st>>>(d_ids, d_dist, uint32_t(nq), int(T), int(k), npad, d_out_ids, d_out_dist);
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace cpb
