// Batched beam search over the flat adjacency, one warp per query, with a fused exact rerank.
//
// Control flow follows SearchEngine::search (include/cphnsw/search/search_engine.hpp:86-193):
// W keeps the `beam` best nodes seen so far, the closest not-yet-expanded member of W is
// expanded next, and the walk ends when every member of W has been expanded (which is when the
// reference's `c.distance > worst.distance` break fires).  Candidates are ordered by the total
// order (distance, id), so the result is independent of the order in which the 32 neighbours of
// a node are examined — that is what lets a warp score a whole adjacency row at once and still
// return exactly what a sequential walk returns.
//
// Metric: the legacy asymmetric CP score (restated at evaluation/debug_estimator.cpp:47-55):
// dist = -sum_r (+-) table[r][index_r], accumulated for r = 0..K-1 in fp32.  The query's K
// rotated vectors (CPQuery::rotated_vecs, include/cphnsw/core/types.hpp:324-337) are staged in
// shared memory (16 KB at K=32, padded dim 128); for large padded dims they stay in global memory.
//
// W lives in shared memory, unsorted, with the current worst member tracked in registers and a
// bit per position marking expanded members; lane l scans positions l, l+32, ...  Visited nodes are tracked in a
// per-warp bitset in global memory that the warp itself returns to all-zero after each query.
// After the walk the beam is sorted by a bitonic network in shared memory; for
// search_and_rerank the best rerank_k are re-scored with -<q,x> (replaces gather_vectors_kernel
// + batch_dot_product_kernel + the host partial_sort of src/cuda/gpu_encoder.cu:605-664) and
// sorted again.
#include <cmath>

#include "common.cuh"

namespace cpb {
namespace {

constexpr uint32_t kFull = 0xffffffffu;
constexpr uint32_t kSeedSlots = 128;  // most seeds a query can have (k_entry <= 100)

struct SearchArgs {
    const float* tables;   // [nq][K][P]
    const float* queries;  // [nq][dim] (rerank only)
    const void* codes;     // [n][K] components
    const uint32_t* adj;   // [n][M]
    const float* vectors;  // [n][dim] (rerank only)
    const uint32_t* entry;     // ids scored for every query before the walk
    const void* entry_codes;   // their codes, gathered contiguously [n_entry][K]
    uint32_t n_entry, n_seed;  // the n_seed best of the scan seed the walk
    uint64_t n;
    uint32_t nq;
    int K, P, dim, M, comp_bytes;
    uint32_t beam, cap, k, rerank_k;  // cap: power of two >= max(32, beam), the size of W's arrays
    uint32_t* visited;  // [total warps][vis_words], all zero between queries
    uint64_t vis_words;
    uint32_t* explist;  // [total warps][exp_cap]
    uint32_t exp_cap;
    uint32_t* out_ids;
    float* out_dist;
    uint32_t* stats;
};

__device__ __forceinline__ bool key_less(float da, uint32_t ia, float db, uint32_t ib) {
    return da < db || (da == db && ia < ib);
}

// asymmetric distance of node `id` against the query table; r ascending, one add per rotation
template <bool U16>
__device__ __forceinline__ float asym_distance(const float* table, const void* codes, uint32_t id, int K,
                                               int P) {
    float acc = 0.0f;
    const int row_bytes = K * (U16 ? 2 : 1);
    const unsigned char* row = static_cast<const unsigned char*>(codes) + size_t(id) * row_bytes;
    if ((row_bytes & 15) == 0) {
        const uint4* r4 = reinterpret_cast<const uint4*>(row);
        int r = 0;
        for (int c = 0; c < row_bytes / 16; ++c) {
            uint4 v = __ldg(r4 + c);
            uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int b = 0; b < (U16 ? 2 : 4); ++b, ++r) {
                    uint32_t comp = U16 ? ((w[i] >> (16 * b)) & 0xffffu) : ((w[i] >> (8 * b)) & 0xffu);
                    float val = table[r * P + int(comp >> 1)];
                    acc = __fadd_rn(acc, (comp & 1u) ? -val : val);
                }
            }
        }
    } else {
        for (int r = 0; r < K; ++r) {
            uint32_t comp = U16 ? uint32_t(reinterpret_cast<const uint16_t*>(row)[r]) : uint32_t(row[r]);
            float val = table[r * P + int(comp >> 1)];
            acc = __fadd_rn(acc, (comp & 1u) ? -val : val);
        }
    }
    return -acc;
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

template <bool U16, bool TABLE_SMEM>
__global__ void search_kernel(SearchArgs a) {
    extern __shared__ __align__(16) unsigned char search_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const size_t table_floats = TABLE_SMEM ? size_t(a.K) * a.P : 0;  // a multiple of 4 when staged
    const size_t dim_pad = (size_t(a.dim) + 3) & ~size_t(3);
    const int cap = int(a.cap);  // power of two >= max(32, beam)
    const int slots = cap >> 5;
    const size_t per_warp = table_floats * 4 + size_t(cap) * 8 + size_t(slots) * 4 + dim_pad * 4;
    unsigned char* mine = search_smem + ((per_warp + 15) & ~size_t(15)) * warp;
    float* table_sm = reinterpret_cast<float*>(mine);
    float* qsm = reinterpret_cast<float*>(mine + table_floats * 4);
    uint32_t* sid = reinterpret_cast<uint32_t*>(qsm + dim_pad);  // W: node ids, position p
    float* sd = reinterpret_cast<float*>(sid + cap);             // W: distances
    uint32_t* expw = reinterpret_cast<uint32_t*>(sd + cap);      // bit p&31 of word p>>5: p expanded

    const uint32_t gwarp = blockIdx.x * warps + warp, total_warps = gridDim.x * warps;
    uint32_t* vis = a.visited + size_t(gwarp) * a.vis_words;
    // per-warp list in HBM: kSeedSlots seed ids, then the ids of expanded nodes
    uint32_t* seedlist = a.explist + size_t(gwarp) * (a.exp_cap + kSeedSlots);
    uint32_t* explist = seedlist + kSeedSlots;
    const uint32_t beam = a.beam;
    const bool scan_mode = a.n_seed < a.n_entry;

    for (uint32_t q = gwarp; q < a.nq; q += total_warps) {
        const float* table = a.tables + size_t(q) * a.K * a.P;
        if (TABLE_SMEM) {
            const float4* src = reinterpret_cast<const float4*>(table);
            float4* dst = reinterpret_cast<float4*>(table_sm);
            for (int i = lane; i < int(table_floats / 4); i += 32) dst[i] = __ldg(src + i);
            table = table_sm;
        }
        if (a.rerank_k) {
            const float* qv = a.queries + size_t(q) * a.dim;
            for (int i = lane; i < int(dim_pad); i += 32) qsm[i] = i < a.dim ? __ldg(qv + i) : 0.0f;
        }
        for (int p = lane; p < cap; p += 32) {
            sd[p] = INFINITY;
            sid[p] = kInvalidNode;
        }
        if (lane < slots) expw[lane] = 0;
        __syncwarp();

        uint32_t count = 0, nexp = 0, nevals = 0, nseeds = 0;
        uint32_t wcap = scan_mode ? a.n_seed : beam;  // capacity of W: the seeds first, then the beam
        bool exp_overflow = false;
        float wd = INFINITY;  // worst member of W once it is full
        uint32_t wi = kInvalidNode;
        int wpos = -1;

        auto recompute_worst = [&]() {
            float ld = 0.0f;
            uint32_t li = 0;
            int lp = -1;
            for (int p = lane; p < int(wcap); p += 32) {
                const float d = sd[p];
                const uint32_t i = sid[p];
                if (lp < 0 || key_less(ld, li, d, i)) {
                    ld = d;
                    li = i;
                    lp = p;
                }
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                const float od = __shfl_xor_sync(kFull, ld, o);
                const uint32_t oi = __shfl_xor_sync(kFull, li, o);
                const int op = __shfl_xor_sync(kFull, lp, o);
                if (op >= 0 && (lp < 0 || key_less(ld, li, od, oi))) {
                    ld = od;
                    li = oi;
                    lp = op;
                }
            }
            wd = ld;
            wi = li;
            wpos = lp;
        };
        auto put = [&](int pos, float d, uint32_t id) {
            if (lane == 0) {
                sd[pos] = d;
                sid[pos] = id;
                expw[pos >> 5] &= ~(1u << (pos & 31));
            }
            __syncwarp();
        };
        // admit one scored candidate per lane into W: W stays the wcap best seen so far
        // (search_engine.hpp:166-176 for a whole row at once)
        auto admit = [&](bool fresh, float dist, uint32_t id) {
            uint32_t m = __ballot_sync(kFull, fresh);
            nevals += __popc(m);
            while (m && count < wcap) {
                const int src = __ffs(m) - 1;
                m &= m - 1;
                put(int(count), __shfl_sync(kFull, dist, src), __shfl_sync(kFull, id, src));
                ++count;
                if (count == wcap) recompute_worst();
            }
            if (m) {
                m &= __ballot_sync(kFull, fresh && key_less(dist, id, wd, wi));
                while (m) {
                    const int src = __ffs(m) - 1;
                    m &= m - 1;
                    const float d = __shfl_sync(kFull, dist, src);
                    const uint32_t i = __shfl_sync(kFull, id, src);
                    if (key_less(d, i, wd, wi)) {
                        put(wpos, d, i);
                        recompute_worst();
                    }
                }
            }
            __syncwarp();
        };
        // offer one node per lane: visited test-and-set, score, admit (search_engine.hpp:153-177)
        auto offer = [&](uint32_t id, bool in_range) {
            // a node listed twice in one row is offered once (the second copy would find it visited)
            const uint32_t grp = __match_any_sync(kFull, id);
            bool fresh = in_range && (__ffs(grp) - 1) == lane;
            if (fresh) {
                const uint32_t word = __ldcg(vis + (id >> 5));
                if ((word >> (id & 31)) & 1u) fresh = false;
                else atomicOr(vis + (id >> 5), 1u << (id & 31));
            }
            float dist = 0.0f;
            if (fresh) dist = asym_distance<U16>(table, a.codes, id, a.K, a.P);
            admit(fresh, dist, id);
        };

        if (scan_mode) {
            // entry scan: score every entry node from the contiguous copy of its code, keep the
            // n_seed best in W; nothing is marked visited until the seeds are known
            for (uint32_t e0 = 0; e0 < a.n_entry; e0 += 32) {
                const uint32_t e = e0 + lane;
                const uint32_t id = e < a.n_entry ? __ldg(a.entry + e) : kInvalidNode;
                const bool ok = id < a.n;
                float dist = 0.0f;
                if (ok) dist = asym_distance<U16>(table, a.entry_codes, e, a.K, a.P);
                admit(ok, dist, id);
            }
            // the seeds are now offered to the walk: mark them visited and remember them for the clean-up
            nseeds = count;
            nevals += nseeds;
            for (uint32_t p = lane; p < nseeds; p += 32) {
                const uint32_t id = sid[p];
                atomicOr(vis + (id >> 5), 1u << (id & 31));
                seedlist[p] = id;
            }
            __syncwarp();
            if (nseeds > beam) {  // a beam narrower than the seed set keeps the best `beam` seeds
                int ns = 32;
                while (ns < int(nseeds)) ns <<= 1;
                warp_sort_smem(sd, sid, ns, lane);
                for (uint32_t p = beam + lane; p < uint32_t(cap); p += 32) {
                    sd[p] = INFINITY;
                    sid[p] = kInvalidNode;
                }
                count = beam;
                __syncwarp();
            }
            wcap = beam;
            if (count == wcap) recompute_worst();
        } else {
            for (uint32_t e0 = 0; e0 < a.n_entry; e0 += 32) {  // search_engine.hpp:105-115
                const uint32_t e = e0 + lane;
                const uint32_t id = e < a.n_entry ? __ldg(a.entry + e) : kInvalidNode;
                offer(id, id < a.n);
            }
        }

        while (true) {
            // closest member of W that has not been expanded (search_engine.hpp:121-123)
            float ld = 0.0f;
            uint32_t li = 0;
            int lp = -1;
            for (int p = lane; p < int(count); p += 32) {
                if ((expw[p >> 5] >> lane) & 1u) continue;
                const float d = sd[p];
                const uint32_t i = sid[p];
                if (lp < 0 || key_less(d, i, ld, li)) {
                    ld = d;
                    li = i;
                    lp = p;
                }
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                const float od = __shfl_xor_sync(kFull, ld, o);
                const uint32_t oi = __shfl_xor_sync(kFull, li, o);
                const int op = __shfl_xor_sync(kFull, lp, o);
                if (op >= 0 && (lp < 0 || key_less(od, oi, ld, li))) {
                    ld = od;
                    li = oi;
                    lp = op;
                }
            }
            if (lp < 0) break;
            if (lane == 0) {
                expw[lp >> 5] |= 1u << (lp & 31);
                if (nexp < a.exp_cap) explist[nexp] = li;
            }
            if (nexp >= a.exp_cap) exp_overflow = true;
            ++nexp;
            __syncwarp();
            const uint32_t* row = a.adj + size_t(li) * a.M;
            for (int m0 = 0; m0 < a.M; m0 += 32) {
                const int j = m0 + lane;
                const uint32_t id = j < a.M ? __ldg(row + j) : kInvalidNode;
                offer(id, id < a.n);
            }
        }

        // return the visited bitset to all-zero: every marked node is an entry id or a neighbour
        // of an expanded node
        if (exp_overflow) {
            for (uint64_t w = lane; w < a.vis_words; w += 32) vis[w] = 0;
        } else {
            if (scan_mode) {
                for (uint32_t p = lane; p < nseeds; p += 32) vis[__ldcg(seedlist + p) >> 5] = 0;
            } else {
                for (uint32_t e = lane; e < a.n_entry; e += 32) {
                    const uint32_t id = __ldg(a.entry + e);
                    if (id < a.n) vis[id >> 5] = 0;
                }
            }
            __syncwarp();
            for (uint32_t x = 0; x < nexp; ++x) {
                const uint32_t node = __ldcg(explist + x);
                const uint32_t* row = a.adj + size_t(node) * a.M;
                for (int j = lane; j < a.M; j += 32) {
                    const uint32_t id = __ldg(row + j);
                    if (id < a.n) vis[id >> 5] = 0;
                }
            }
        }
        __syncwarp();

        // sort W ascending; positions past `count` hold (+inf, no node)
        int nsort = 32;
        while (nsort < int(count)) nsort <<= 1;
        warp_sort_smem(sd, sid, nsort, lane);

        if (a.rerank_k) {
            const uint32_t ncand = min(a.rerank_k, count);
            const int g = lane >> 3, j = lane & 7;
            const bool vec4 = (a.dim & 3) == 0;
            for (uint32_t c0 = 0; c0 < ncand; c0 += 4) {
                const uint32_t c = c0 + g;
                float acc = 0.0f;
                if (c < ncand) {
                    const float* x = a.vectors + size_t(sid[c]) * a.dim;
                    if (vec4) {
                        for (int i = 4 * j; i < a.dim; i += 32) {
                            const float4 xv = __ldg(reinterpret_cast<const float4*>(x + i));
                            const float4 qv = *reinterpret_cast<const float4*>(qsm + i);
                            acc = fmaf(xv.x, qv.x, acc);
                            acc = fmaf(xv.y, qv.y, acc);
                            acc = fmaf(xv.z, qv.z, acc);
                            acc = fmaf(xv.w, qv.w, acc);
                        }
                    } else {
                        for (int i = j; i < a.dim; i += 8) acc = fmaf(__ldg(x + i), qsm[i], acc);
                    }
                }
                acc += __shfl_xor_sync(kFull, acc, 4);
                acc += __shfl_xor_sync(kFull, acc, 2);
                acc += __shfl_xor_sync(kFull, acc, 1);
                if (c < ncand && j == 0) sd[c] = -acc;
            }
            nsort = 32;
            while (nsort < int(ncand)) nsort <<= 1;
            for (int pos = int(ncand) + lane; pos < nsort; pos += 32) {
                sd[pos] = INFINITY;
                sid[pos] = kInvalidNode;
            }
            __syncwarp();
            warp_sort_smem(sd, sid, nsort, lane);
        }

        uint32_t* oid = a.out_ids + size_t(q) * a.k;
        float* od = a.out_dist + size_t(q) * a.k;
        for (uint32_t pos = lane; pos < a.k; pos += 32) {
            const bool have = pos < uint32_t(nsort) && sid[pos] != kInvalidNode;
            oid[pos] = have ? sid[pos] : kInvalidNode;
            od[pos] = have ? sd[pos] : INFINITY;
        }
        if (a.stats && lane == 0) {
            a.stats[2 * size_t(q)] = nexp;
            a.stats[2 * size_t(q) + 1] = nevals;
        }
        __syncwarp();
    }
}

__global__ void gather_rows_kernel(const unsigned char* __restrict__ src, int row_bytes,
                                   const uint32_t* __restrict__ ids, uint32_t n_ids, uint64_t n,
                                   unsigned char* __restrict__ dst) {
    const uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= uint64_t(n_ids) * row_bytes) return;
    const uint32_t id = ids[i / row_bytes];
    dst[i] = id < n ? src[uint64_t(id) * row_bytes + i % row_bytes] : 0;
}

struct LaunchCfg {
    uint32_t cap;
    int warps;
    size_t per_warp;
    bool table_smem;
};

LaunchCfg pick_cfg(const cphnsw_b200_index* h, uint32_t beam) {
    LaunchCfg c;
    c.cap = 32;
    while (c.cap < beam || c.cap < h->k_entry) c.cap <<= 1;
    const size_t table_bytes = size_t(h->K) * h->P * 4;
    c.table_smem = table_bytes <= 32 * 1024 && (table_bytes % 16) == 0;
    const size_t dim_pad = (size_t(h->dim) + 3) & ~size_t(3);
    size_t per_warp = (c.table_smem ? table_bytes : 0) + size_t(c.cap) * 8 + size_t(c.cap / 32) * 4 + dim_pad * 4;
    per_warp = (per_warp + 15) & ~size_t(15);
    const size_t budget = 220 * 1024;
    int w = int(budget / per_warp);
    if (w > 16) w = 16;
    if (w < 1) w = 1;
    c.warps = w;
    c.per_warp = per_warp;
    return c;
}

}  // namespace

int gather_entry_codes(cphnsw_b200_index* h, cudaStream_t st) {
    const int row_bytes = int(h->K * h->comp_bytes);
    CPB_TRY(h->d_entry_codes.reserve(size_t(h->n_entry) * row_bytes + 16));
    const uint64_t total = uint64_t(h->n_entry) * row_bytes;
    if (total) {
        gather_rows_kernel<<<unsigned((total + 255) / 256), 256, 0, st>>>(
            h->d_codes.as<unsigned char>(), row_bytes, h->d_entry.as<uint32_t>(), h->n_entry, h->n,
            h->d_entry_codes.as<unsigned char>());
        h->launches++;
        CPB_CUDA(cudaGetLastError());
    }
    return 0;
}

int prepare_search_scratch(cphnsw_b200_index* h, uint32_t beam) {
    const size_t total_warps = size_t(h->sm_count) * 16;  // the most warps a launch ever uses
    const size_t vis_words = (h->n + 31) / 32;
    const size_t vis_bytes = total_warps * vis_words * 4;
    if (vis_bytes > h->d_visited.bytes || !h->d_visited.p) {
        CPB_TRY(h->d_visited.reserve(vis_bytes));
        CPB_CUDA(cudaMemset(h->d_visited.p, 0, h->d_visited.bytes));
    }
    const size_t exp_cap = size_t(4) * beam + 64;
    CPB_TRY(h->d_explist.reserve(total_warps * (exp_cap + kSeedSlots) * 4));
    return 0;
}

int launch_search(cphnsw_b200_index* h, const float* d_q, const float* d_tables, uint64_t nq, uint32_t k,
                  uint32_t beam, uint32_t rerank_k, uint32_t* d_ids, float* d_dists, uint32_t* d_stats,
                  cudaStream_t st) {
    if (nq == 0) return 0;
    if (beam > 1024) {
        set_error("search: beam width max(ef, k, rerank_k) must be <= 1024 (got %u)", beam);
        return CPHNSW_B200_E_INVALID;
    }
    if (nq > 0xffffffffull) {
        set_error("search: at most 2^32-1 queries per call");
        return CPHNSW_B200_E_INVALID;
    }
    CPB_TRY(prepare_search_scratch(h, beam));
    LaunchCfg c = pick_cfg(h, beam);
    SearchArgs a;
    a.tables = d_tables;
    a.queries = d_q;
    a.codes = h->d_codes.p;
    a.adj = h->d_adj.as<uint32_t>();
    a.vectors = h->d_vectors.as<float>();
    a.entry = h->d_entry.as<uint32_t>();
    a.entry_codes = h->d_entry_codes.p;
    a.n_entry = h->n_entry;
    a.n_seed = h->k_entry;
    a.n = h->n;
    a.nq = uint32_t(nq);
    a.K = int(h->K);
    a.P = int(h->P);
    a.dim = int(h->dim);
    a.M = int(h->M);
    a.comp_bytes = int(h->comp_bytes);
    a.beam = beam;
    a.cap = c.cap;
    a.k = k;
    a.rerank_k = rerank_k;
    a.visited = h->d_visited.as<uint32_t>();
    a.vis_words = (h->n + 31) / 32;
    a.explist = h->d_explist.as<uint32_t>();
    a.exp_cap = 4 * beam + 64;
    a.out_ids = d_ids;
    a.out_dist = d_dists;
    a.stats = d_stats;
    const unsigned grid = unsigned(h->sm_count);
    const bool u16 = h->comp_bytes == 2;
    LaunchTimer timer(h, kKernelSearch, st);

#define CPB_SEARCH(U, T)                                                                                   \
    do {                                                                                                   \
        cudaFuncAttributes fa;                                                                             \
        CPB_CUDA(cudaFuncGetAttributes(&fa, search_kernel<U, T>));                                         \
        int maxw = 65536 / (((fa.numRegs + 7) & ~7) * 32);                                                 \
        int w = c.warps < maxw ? c.warps : maxw;                                                           \
        size_t smem = c.per_warp * w;                                                                      \
        CPB_CUDA(cudaFuncSetAttribute(search_kernel<U, T>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                      int(smem)));                                                         \
        search_kernel<U, T><<<grid, w * 32, smem, st>>>(a);                                                \
    } while (0)
    if (u16 && c.table_smem) CPB_SEARCH(true, true);
    else if (u16) CPB_SEARCH(true, false);
    else if (c.table_smem) CPB_SEARCH(false, true);
    else CPB_SEARCH(false, false);
#undef CPB_SEARCH
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace cpb
