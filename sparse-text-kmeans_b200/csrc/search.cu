// Batched beam search over the flat adjacency, one warp per query, with a fused exact rerank.
//
// Control flow follows SearchEngine::search (include/cphnsw/search/search_engine.hpp:86-193):
// W keeps the `beam` best nodes seen so far, the closest not-yet-expanded member of W is
// expanded next, and the walk ends when every member of W has been expanded (which is when the
// reference's `c.distance > worst.distance` break fires).  Candidates are ordered by the total
// order (distance, id), so W after an expansion is the `beam` best of everything seen, whatever
// the order in which the 32 neighbours of a node are examined — that is what lets a warp score a
// whole adjacency row at once and still return exactly what a sequential walk returns.
//
// Metric: the legacy asymmetric CP score (restated at evaluation/debug_estimator.cpp:47-55):
// dist = -sum_r (+-) table[r][index_r] in fp32.  The K terms are added in a fixed balanced-tree
// order (per block of 32 rotations: pairs 16 apart, then 8, 4, 2, 1; blocks added in sequence),
// which is the order a warp shuffle reduction produces; the same order is used when one lane
// scores a node alone, so every path yields the same float.  (The reference's scalar form adds
// r = 0..K-1 in sequence and its SIMD batch form in yet another order; the two agree to 1e-5,
// evaluation/qa_protocol.cpp:168-244.)  The query's K rotated vectors (CPQuery::rotated_vecs,
// include/cphnsw/core/types.hpp:324-337) are staged in shared memory (16 KB at K=32, padded dim
// 128); for large padded dims they stay in global memory.
//
// W lives in shared memory, sorted ascending, the "expanded" flag in the top bit of the id; a
// cursor tracks the first unexpanded member, an admission finds its rank with a two-round 32-ary
// search and shifts the tail up by one.  Visited nodes are tracked in a per-warp array of one
// byte per node in global memory holding the number ("epoch") of the last query of that warp
// that visited the node, so nothing has to be cleared between queries (the array is zeroed when
// the 8-bit epoch wraps).  The adjacency row and the visited bytes of the node expected to be
// expanded next are loaded one expansion ahead.  For search_and_rerank the
// best rerank_k are re-scored with -<q,x> (replaces gather_vectors_kernel + batch_dot_product_kernel
// + the host partial_sort of src/cuda/gpu_encoder.cu:605-664) and sorted by a bitonic network.
#include <cmath>

#include "search_common.cuh"

namespace cpb {
namespace {

using namespace srch;

template <bool U16, bool TABLE_SMEM, bool SYM>
__global__ void search_kernel(SearchArgs a) {
    extern __shared__ __align__(16) unsigned char search_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const size_t table_floats = TABLE_SMEM ? size_t(a.K) * a.P : 0;  // a multiple of 4 when staged
    const size_t dim_pad = a.qsm_floats;  // floats of the query-vector / query-code area (multiple of 4)
    const int cap = int(a.cap);
    unsigned char* mine = search_smem + size_t(a.per_warp_smem) * warp;
    float* table_sm = reinterpret_cast<float*>(mine);
    float* qsm = reinterpret_cast<float*>(mine + table_floats * 4);
    uint32_t* sid = reinterpret_cast<uint32_t*>(qsm + dim_pad);  // W: node ids (+ expanded bit), ascending
    float* sd = reinterpret_cast<float*>(sid + cap);             // W: distances

    const uint32_t gwarp = blockIdx.x * warps + warp;
    uint8_t* vis = a.visited + size_t(gwarp) * a.vis_stride;
    uint32_t epoch = a.epochs[gwarp];  // 1..255; 0 marks "never visited"
    const uint32_t beam = a.beam;
    const bool scan_mode = a.scan_only || a.n_seed < a.n_entry;
    const int row_bytes = a.K * (U16 ? 2 : 1);
    const bool coop_ok = !SYM && a.K <= 64;
    const bool two_blocks = a.K > 32;  // a lane owns two rotations in the whole-warp scoring
    const unsigned char* qcode_sm = reinterpret_cast<const unsigned char*>(qsm + a.qvec_floats);  // symmetric metric only
    // binary-code mode: the query's sign bits packed 32 per word, behind its code
    uint32_t* qpacked_sm = reinterpret_cast<uint32_t*>(qsm + a.qvec_floats + ((row_bytes + 15) / 16) * 4);

    // queries are handed out one at a time from a global counter, so that warps that draw short
    // walks take more of them
    while (true) {
        uint32_t q = 0;
        if (lane == 0) q = atomicAdd(a.next_query, 1u);
        q = __shfl_sync(kFull, q, 0);
        if (q >= a.nq) break;
        const float* table = SYM ? nullptr : a.tables + size_t(q) * a.K * a.P;
        if (SYM) {
            const unsigned char* src = static_cast<const unsigned char*>(a.qcodes) + size_t(q) * row_bytes;
            for (int i = lane; i < row_bytes; i += 32) reinterpret_cast<unsigned char*>(qsm + a.qvec_floats)[i] = src[i];
            if (a.packed) {
                __syncwarp();
                for (int w = 0; w < a.packed_words; ++w) {
                    const int r = 32 * w + lane;
                    const uint32_t word = __ballot_sync(kFull, r < a.K && (qcode_sm[r * (U16 ? 2 : 1)] & 1u));
                    if (lane == 0) qpacked_sm[w] = word;
                }
            }
        }
        if (TABLE_SMEM && !SYM) {
            const float4* src = reinterpret_cast<const float4*>(table);
            float4* dst = reinterpret_cast<float4*>(table_sm);
            for (int i = lane; i < int(table_floats / 4); i += 32) dst[i] = __ldg(src + i);
            table = table_sm;
        }
        if (a.rerank_k) {
            const float* qv = a.queries + size_t(q) * a.dim;
            for (int i = lane; i < int(a.qvec_floats); i += 32) qsm[i] = i < a.dim ? __ldg(qv + i) : 0.0f;
        }
        for (int p = lane; p < cap; p += 32) {
            sd[p] = INFINITY;
            sid[p] = kInvalidNode;
        }
        if (++epoch == 256) {  // the 8-bit epoch wraps: forget every earlier query
            uint4* v4 = reinterpret_cast<uint4*>(vis);
            for (uint64_t i = lane; i < a.vis_stride / 16; i += 32) v4[i] = make_uint4(0u, 0u, 0u, 0u);
            epoch = 1;
        }
        __syncwarp();

        uint32_t count = 0, nexp = 0, nevals = 0;
        uint32_t wcap = scan_mode ? a.n_seed : beam;  // capacity of W: the seeds first, then the beam
        uint32_t cur = 0;                             // first unexpanded position of W (== count when none)
        float wd = INFINITY;  // worst member of W once it is full
        uint32_t wi = kInvalidNode;

        // one lane scores one node (row `row` of `code_base`) under the kernel's metric
        auto score_lane = [&](const void* code_base, uint32_t row) -> float {
            if (SYM) {
                if (a.packed && code_base == a.codes)  // the walk (the entry scan reads its own contiguous copy of the codes)
                    return packed_distance_lane(qpacked_sm, a.packed, row, a.packed_words, a.resid_kp, a.resid_mul);
                return sym_distance_lane<U16>(qcode_sm, code_base, row, a.K, a.resid_kp, a.resid_mul);
            }
            return asym_distance_lane<U16>(table, code_base, row, a.K, a.P);
        };
        // Admission of (d, id), known to every lane: W stays the wcap best seen so far, sorted
        // (search_engine.hpp:166-176).
        auto try_admit = [&](float d, uint32_t id) {
            if (count == wcap && !key_less(d, id, wd, wi)) return;
            // rank = number of members below (d, id): two rounds of a 32-ary search
            uint32_t p = 0;
            if (count) {
                const uint32_t stride = (count + 31) >> 5;
                const uint32_t e = min(count, (uint32_t(lane) + 1) * stride) - 1;
                const bool in = uint32_t(lane) * stride < count;
                const bool less = in && key_less(sd[e], sid[e] & kIdMask, d, id);
                const uint32_t b = __popc(__ballot_sync(kFull, less));  // blocks entirely below
                // second round inside block b: one pass of 32 members, more for a beam wider than 1,024
                uint32_t inside = 0;
                for (uint32_t o = 0; o < stride; o += 32) {
                    const uint32_t j = b * stride + o + lane;
                    const bool less2 = b < 32 && o + uint32_t(lane) < stride && j < count && key_less(sd[j], sid[j] & kIdMask, d, id);
                    inside += __popc(__ballot_sync(kFull, less2));
                }
                p = min(count, b * stride) + inside;
            }
            // shift [p, end) up by one, highest chunk first; a full W drops its last member
            const int end = int(count == wcap ? wcap - 1 : count);
            for (int top = end; top > int(p); top -= 32) {
                const int i = top - 1 - lane;
                const bool act = i >= int(p);
                float md = 0.0f;
                uint32_t mi = 0;
                if (act) {
                    md = sd[i];
                    mi = sid[i];
                }
                __syncwarp();
                if (act) {
                    sd[i + 1] = md;
                    sid[i + 1] = mi;
                }
                __syncwarp();
            }
            if (lane == 0) {
                sd[p] = d;
                sid[p] = id;
            }
            __syncwarp();
            if (count < wcap) ++count;
            if (p <= cur) cur = p;
            if (count == wcap) {
                wd = sd[wcap - 1];
                wi = sid[wcap - 1] & kIdMask;
            }
        };

        // offer one node per lane: visited test-and-set, score, admit (search_engine.hpp:153-177)
        // `have_vis`: the node's visited byte is already in `vbyte` (loaded one expansion ahead);
        // `ahead()` runs once the visited marks of this row are made and its code loads issued
        auto offer = [&](uint32_t id, bool in_range, bool have_vis, uint32_t vbyte, auto&& ahead) {
            // a node listed twice in one row is offered once (the second copy would find it visited)
            bool fresh = in_range;
            if (!a.rows_distinct) {  // every lane takes part in the match, in range or not
                const uint32_t grp = __match_any_sync(kFull, id);
                fresh = fresh && (__ffs(grp) - 1) == lane;
            }
            if (fresh) {
                if (!have_vis) vbyte = __ldcg(vis + id);
                if (vbyte == epoch) fresh = false;
                else vis[id] = uint8_t(epoch);
            }
            uint32_t m = __ballot_sync(kFull, fresh);  // (orders the marks before anything loaded below)
            const int nf = __popc(m);
            nevals += nf;
            if (nf == 0) {
                ahead();
                return;
            }
            if (coop_ok && nf <= kCoopMax) {
                // few fresh nodes: the whole warp scores each of them, one rotation per lane
                uint32_t cid[kCoopMax], comp[kCoopMax], comph[kCoopMax];
#pragma unroll
                for (int f = 0; f < kCoopMax; ++f) {
                    cid[f] = kInvalidNode;
                    comp[f] = 0;
                    comph[f] = 0;
                    if (f < nf) {
                        const int src = __ffs(m) - 1;
                        m &= m - 1;
                        cid[f] = __shfl_sync(kFull, id, src);
                        const unsigned char* crow = static_cast<const unsigned char*>(a.codes) + size_t(cid[f]) * row_bytes;
                        if (lane < a.K) comp[f] = load_component<U16>(crow, lane);
                        if (32 + lane < a.K) comph[f] = load_component<U16>(crow, 32 + lane);
                    }
                }
                ahead();
#pragma unroll
                for (int f = 0; f < kCoopMax; ++f) {
                    if (f < nf) {
                        const float d = two_blocks ? asym_distance_coop2(table, a.K, a.P, comp[f], comph[f], lane)
                                                   : asym_distance_coop(table, a.K, a.P, comp[f], lane);
                        try_admit(d, cid[f]);
                    }
                }
            } else {
                ahead();
                float dist = 0.0f;
                if (fresh) dist = score_lane(a.codes, id);
                if (count == wcap) m &= __ballot_sync(kFull, fresh && key_less(dist, id, wd, wi));
                while (m) {
                    const int src = __ffs(m) - 1;
                    m &= m - 1;
                    try_admit(__shfl_sync(kFull, dist, src), __shfl_sync(kFull, id, src));
                }
            }
        };
        auto nothing = [] {};

        if (scan_mode) {
            // entry scan: score every entry node from the contiguous copy of its code, keep the
            // n_seed best in W; nothing is marked visited until the seeds are known
            for (uint32_t e0 = 0; e0 < a.n_entry; e0 += 32) {
                const uint32_t e = e0 + lane;
                if (e + 32 < a.n_entry) {  // pull the next batch towards L1 while this one is scored
                    if (a.entry) prefetch_l1(a.entry + e + 32);
                    if (a.entry_codes)  // (null for a brute-force scan in binary-code mode, which reads the packed bits)
                        prefetch_l1(static_cast<const unsigned char*>(a.entry_codes) + size_t(e + 32) * row_bytes);
                }
                const uint32_t id = e < a.n_entry ? (a.entry ? __ldg(a.entry + e) : e) : kInvalidNode;
                const bool ok = id < a.n;
                float dist = 0.0f;
                if (ok) dist = score_lane(a.entry_codes, e);
                uint32_t m = __ballot_sync(kFull, ok);
                nevals += __popc(m);
                if (count == wcap) m &= __ballot_sync(kFull, ok && key_less(dist, id, wd, wi));
                while (m) {
                    const int src = __ffs(m) - 1;
                    m &= m - 1;
                    try_admit(__shfl_sync(kFull, dist, src), __shfl_sync(kFull, id, src));
                }
            }
            if (a.scan_only) {
                cur = count;  // nothing to expand: the best of the scan are the result
            } else {
            // the seeds are now offered to the walk: mark them visited
            const uint32_t nseeds = count;
            nevals += nseeds;
            for (uint32_t p = lane; p < nseeds; p += 32) vis[sid[p]] = uint8_t(epoch);
            if (nseeds > beam) {  // a beam narrower than the seed set keeps the best `beam` seeds
                __syncwarp();
                for (uint32_t p = beam + lane; p < uint32_t(cap); p += 32) {
                    sd[p] = INFINITY;
                    sid[p] = kInvalidNode;
                }
                count = beam;
            }
            __syncwarp();
            wcap = beam;
            cur = 0;
            if (count == wcap) {
                wd = sd[wcap - 1];
                wi = sid[wcap - 1] & kIdMask;
            }
            }
        } else {
            for (uint32_t e0 = 0; e0 < a.n_entry; e0 += 32) {  // search_engine.hpp:105-115
                const uint32_t e = e0 + lane;
                const uint32_t id = e < a.n_entry ? __ldg(a.entry + e) : kInvalidNode;
                offer(id, id < a.n, false, 0u, nothing);
            }
        }

        // row and visited bytes loaded one expansion ahead for the node predicted to be next
        uint32_t pre_node = kInvalidNode, pre_id = kInvalidNode, pre_vis = 0;
        bool pre_vis_ok = false;
        const bool single_row = a.M <= 32;  // the visited bytes stay valid only if no later marks intervene
        while (cur < count) {
            // closest member of W that has not been expanded (search_engine.hpp:121-123)
            const uint32_t node = sid[cur] & kIdMask;
            __syncwarp();
            if (lane == 0) sid[cur] = node | kExpanded;
            ++nexp;
            __syncwarp();
            // advance the cursor to the next unexpanded member
            uint32_t nxt = cur + 1;
            while (nxt < count) {
                const uint32_t j = nxt + lane;
                const uint32_t un = __ballot_sync(kFull, j < count && !(sid[j] & kExpanded));
                if (un) {
                    nxt += __ffs(un) - 1;
                    break;
                }
                nxt += 32;
            }
            cur = min(nxt, count);
            const uint32_t* row = a.adj + size_t(node) * a.M;
            const bool hit = node == pre_node;
            const uint32_t first = hit ? pre_id : (lane < a.M ? __ldg(row + lane) : kInvalidNode);
            const bool have_vis = hit && pre_vis_ok;
            const uint32_t first_vis = pre_vis;
            // predict the next node (the cursor, unless this expansion admits something closer)
            // and start loading its row now; its visited bytes follow once this row's marks are made
            pre_node = cur < count ? (sid[cur] & kIdMask) : kInvalidNode;
            pre_id = (pre_node != kInvalidNode && lane < a.M) ? __ldg(a.adj + size_t(pre_node) * a.M + lane) : kInvalidNode;
            pre_vis_ok = false;
            offer(first, first < a.n, have_vis, first_vis, [&] {
                if (single_row) {
                    __syncwarp();  // this row's marks are ordered before the bytes read ahead
                    pre_vis = pre_id < a.n ? uint32_t(__ldcg(vis + pre_id)) : 0u;
                    pre_vis_ok = true;
                }
            });
            for (int m0 = 32; m0 < a.M; m0 += 32) {
                const int j = m0 + lane;
                const uint32_t id = j < a.M ? __ldg(row + j) : kInvalidNode;
                offer(id, id < a.n, false, 0u, nothing);
            }
        }

        // W is sorted already; drop the expanded flags
        for (uint32_t p = lane; p < count; p += 32) sid[p] &= kIdMask;
        __syncwarp();
        int nsort = 32;
        while (nsort < int(count)) nsort <<= 1;

        if (a.rerank_k) {
            const uint32_t ncand = min(a.rerank_k, count);
            const int g = lane >> 3, j = lane & 7;
            const bool vec4 = (a.dim & 3) == 0;
#pragma unroll 4
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
            if (a.k <= kSelectMax) {  // the few results wanted are picked out; everything behind them stays unsorted
                nsort = int(ncand);
                __syncwarp();
                warp_select_smem(sd, sid, nsort, int(a.k), lane);
            } else {
                nsort = 32;
                while (nsort < int(ncand)) nsort <<= 1;
                for (int pos = int(ncand) + lane; pos < nsort; pos += 32) {
                    sd[pos] = INFINITY;
                    sid[pos] = kInvalidNode;
                }
                __syncwarp();
                warp_sort_smem(sd, sid, nsort, lane);
            }
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
    if (lane == 0) a.epochs[gwarp] = epoch;
}

__global__ void gather_rows_kernel(const unsigned char* __restrict__ src, int row_bytes,
                                   const uint32_t* __restrict__ ids, uint32_t n_ids, uint64_t n,
                                   unsigned char* __restrict__ dst) {
    const uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= uint64_t(n_ids) * row_bytes) return;
    const uint32_t id = ids[i / row_bytes];
    dst[i] = id < n ? src[uint64_t(id) * row_bytes + i % row_bytes] : 0;
}

// one warp per adjacency row (M <= 32): a valid id that appears twice raises the flag
__global__ void adjacency_dup_kernel(const uint32_t* __restrict__ adj, uint64_t n, int M, uint32_t* __restrict__ flag) {
    const int lane = threadIdx.x & 31;
    const uint64_t row = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (row >= n) return;
    const uint32_t id = lane < M ? adj[row * M + lane] : kInvalidNode;
    const uint32_t grp = __match_any_sync(kFull, id);
    const bool dup = id < n && (__ffs(grp) - 1) != lane;
    if (__ballot_sync(kFull, dup) && lane == 0) atomicOr(flag, 1u);
}

struct LaunchCfg {
    uint32_t cap;
    int warps;
    size_t per_warp;
    size_t qsm_floats, qvec_floats;
    bool table_smem;
};

LaunchCfg pick_cfg(const cphnsw_b200_index* h, uint32_t beam, bool sym) {
    LaunchCfg c;
    c.cap = 32;
    while (c.cap < beam || c.cap < h->k_entry) c.cap <<= 1;
    const size_t table_bytes = size_t(h->K) * h->P * 4;
    c.table_smem = !sym && h->search_table_smem && table_bytes <= 32 * 1024 && (table_bytes % 16) == 0;
    const size_t qvec = (size_t(h->dim) + 3) & ~size_t(3);
    // under the symmetric metric the query code follows the query vector
    size_t dim_pad = qvec + (sym ? ((size_t(h->K) * h->comp_bytes + 15) / 16) * 4 : 0);
    if (sym) dim_pad += (((size_t(h->K) + 31) / 32 * 4 + 15) / 16) * 4;  // and its sign bits, packed (binary-code mode)
    c.qvec_floats = qvec;
    size_t per_warp = (c.table_smem ? table_bytes : 0) + size_t(c.cap) * 8 + dim_pad * 4;
    per_warp = (per_warp + 15) & ~size_t(15);
    const size_t budget = 226 * 1024;  // of the 227 KB a block may use
    int w = int(budget / per_warp);
    if (w > 16) w = 16;
    if (w < 1) w = 1;
    c.warps = w;
    c.per_warp = per_warp;
    c.qsm_floats = dim_pad;
    return c;
}

}  // namespace

// two-warps-per-query kernel (search_team.cu)
size_t search_team_extra_smem();
int launch_search_team(cphnsw_b200_index* h, SearchArgs a, size_t per_team, int narrow_blocks, cudaStream_t st);

// sign bits of every node, 32 per word: bit b of word w = bit 0 of component 32 * w + b (binary-code mode)
__global__ void pack_walk_codes_kernel(const unsigned char* __restrict__ codes, uint64_t n, int K, int comp_bytes, int words,
                                       uint32_t* __restrict__ out) {
    const uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= n * uint64_t(words)) return;
    const uint64_t node = t / words;
    const int w = int(t % words);
    const unsigned char* row = codes + node * uint64_t(K) * comp_bytes;
    uint32_t bits = 0;
    for (int b = 0; b < 32 && w * 32 + b < K; ++b)
        if (row[size_t(w * 32 + b) * comp_bytes] & 1u) bits |= 1u << b;
    out[t] = bits;
}

// the inverse: one component (0 or 1) per bit
__global__ void unpack_walk_codes_kernel(const uint32_t* __restrict__ packed, uint64_t n, int K, int comp_bytes, int words,
                                         unsigned char* __restrict__ codes) {
    const uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= n * uint64_t(K)) return;
    const uint64_t node = t / K;
    const int r = int(t % K);
    const uint32_t bit = (packed[node * words + (r >> 5)] >> (r & 31)) & 1u;
    unsigned char* c = codes + t * comp_bytes;
    c[0] = (unsigned char)bit;
    if (comp_bytes == 2) c[1] = 0;
}

int ensure_codes(cphnsw_b200_index* h, cudaStream_t st) {
    if (!h->codes_released) return 0;
    const size_t rb = size_t(h->K) * h->comp_bytes;
    CPB_TRY(h->d_codes.reserve(size_t(h->n) * rb + 16));
    const uint64_t total = uint64_t(h->n) * h->K;
    if (total) {
        unpack_walk_codes_kernel<<<unsigned((total + 255) / 256), 256, 0, st>>>(h->d_packed.as<uint32_t>(), h->n, int(h->K),
                                                                               int(h->comp_bytes), h->packed_words,
                                                                               h->d_codes.as<unsigned char>());
        h->launches++;
        CPB_CUDA(cudaGetLastError());
    }
    h->codes_released = false;
    return 0;
}

// after the stored codes or the entry ids change: the contiguous copy of the entry nodes' codes and, in binary-code
// mode, the packed sign bits the walk reads
int gather_entry_codes(cphnsw_b200_index* h, cudaStream_t st) {
    CPB_TRY(ensure_codes(h, st));
    h->packed_words = 0;
    if (h->binary_codes && h->n) {
        const int words = int((h->K + 31) / 32);
        CPB_TRY(h->d_packed.reserve(size_t(h->n) * words * 4 + 16));
        const uint64_t total = uint64_t(h->n) * words;
        pack_walk_codes_kernel<<<unsigned((total + 255) / 256), 256, 0, st>>>(h->d_codes.as<unsigned char>(), h->n, int(h->K),
                                                                             int(h->comp_bytes), words, h->d_packed.as<uint32_t>());
        h->launches++;
        CPB_CUDA(cudaGetLastError());
        h->packed_words = words;
    }
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

// dst[i] = row ids[i] of src (rows of row_bytes bytes; ids >= n give zero rows)
int gather_rows(cphnsw_b200_index* h, const void* src, size_t row_bytes, const uint32_t* d_ids, uint32_t n_ids, void* dst,
                cudaStream_t st) {
    const uint64_t total = uint64_t(n_ids) * row_bytes;
    if (total == 0) return 0;
    gather_rows_kernel<<<unsigned((total + 255) / 256), 256, 0, st>>>(static_cast<const unsigned char*>(src), int(row_bytes),
                                                                     d_ids, n_ids, h->n, static_cast<unsigned char*>(dst));
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

int scan_adjacency_rows(cphnsw_b200_index* h, cudaStream_t st) {
    h->adj_rows_distinct = 0;
    if (h->n == 0 || h->M > 32 || !h->d_adj.p) return 0;  // wider rows: the search dedupes each batch of 32
    uint32_t* flag = h->d_status.as<uint32_t>() + 2;
    CPB_CUDA(cudaMemsetAsync(flag, 0, 4, st));
    const uint64_t threads = h->n * 32;
    adjacency_dup_kernel<<<unsigned((threads + 255) / 256), 256, 0, st>>>(h->d_adj.as<uint32_t>(), h->n, int(h->M), flag);
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    uint32_t dup = 1;
    CPB_CUDA(cudaMemcpyAsync(&dup, flag, 4, cudaMemcpyDeviceToHost, st));
    CPB_CUDA(cudaStreamSynchronize(st));
    h->adj_rows_distinct = dup == 0;
    return 0;
}

int prepare_search_scratch(cphnsw_b200_index* h, SearchCtx& cx, cudaStream_t st) {
    // the most slots a launch of this context uses: one per query (narrow) or 16 per SM (wide)
    const size_t slots = cx.wide ? size_t(h->sm_count) * 16 : size_t(kNarrowQueries);
    size_t stride = (size_t(h->n) + 15) & ~size_t(15);
    // an array laid out for more nodes than the index holds stays valid (an index that grows by
    // incremental insertion gets a quarter of slack so that not every insertion reallocates)
    if (cx.d_visited.p && cx.vis_stride >= stride && slots * cx.vis_stride <= cx.d_visited.bytes) return 0;
    if (cx.d_visited.p) stride = (stride + stride / 4 + 15) & ~size_t(15);
    CPB_TRY(cx.d_visited.reserve(slots * stride));
    CPB_CUDA(cudaMemsetAsync(cx.d_visited.p, 0, cx.d_visited.bytes, st));
    CPB_TRY(cx.d_epochs.reserve(slots * 4));  // per-slot epoch counters
    CPB_CUDA(cudaMemsetAsync(cx.d_epochs.p, 0, cx.d_epochs.bytes, st));
    cx.vis_stride = stride;
    cx.vis_slots = slots;
    return 0;
}

void drop_search_scratch(cphnsw_b200_index* h) {
    std::lock_guard<std::mutex> lock(h->ctx_mu);
    for (auto& c : h->ctxs) {
        c->d_visited.release();
        c->vis_stride = 0;
    }
}

int launch_search(cphnsw_b200_index* h, SearchCtx& cx, const float* d_q, const float* d_tables, uint64_t nq, uint32_t k,
                  uint32_t beam, uint32_t rerank_k, uint32_t* d_ids, float* d_dists, uint32_t* d_stats,
                  cudaStream_t st, const void* d_qcodes, int scan_only) {
    const bool sym = d_qcodes != nullptr;  // symmetric code-distance walk (search_multiprobe)
    if (nq == 0) return 0;
    if (beam > kMaxBeam) {
        set_error("search: beam width max(ef, k, rerank_k) must be <= %u (got %u)", kMaxBeam, beam);
        return CPHNSW_B200_E_INVALID;
    }
    if (nq > 0xffffffffull) {
        set_error("search: at most 2^32-1 queries per call");
        return CPHNSW_B200_E_INVALID;
    }
    if (!cx.wide && nq > kNarrowQueries) {
        set_error("search: internal error (a narrow context was given %llu queries)", (unsigned long long)nq);
        return CPHNSW_B200_E_STATE;
    }
    CPB_TRY(prepare_search_scratch(h, cx, st));
    LaunchCfg c = pick_cfg(h, beam, sym);
    SearchArgs a;
    a.qcodes = d_qcodes;
    a.qsm_floats = uint32_t(c.qsm_floats);
    a.qvec_floats = uint32_t(c.qvec_floats);
    a.tables = d_tables;
    a.queries = d_q;
    a.codes = h->d_codes.p;
    a.packed = (sym && h->binary_codes && h->packed_words) ? h->d_packed.as<uint32_t>() : nullptr;
    a.packed_words = h->packed_words;
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
    a.per_warp_smem = uint32_t(c.per_warp);
    a.k = k;
    a.rerank_k = rerank_k;
    a.visited = cx.d_visited.as<uint8_t>();
    a.vis_stride = cx.vis_stride;
    a.epochs = cx.d_epochs.as<uint32_t>();
    a.out_ids = d_ids;
    a.out_dist = d_dists;
    a.stats = d_stats;
    a.next_query = cx.d_counter.as<uint32_t>();
    a.rows_distinct = h->adj_rows_distinct;
    a.scan_only = scan_only;
    a.resid_kp = h->residual_bits ? int(h->K - h->residual_bits) : 0;
    a.resid_mul = h->residual_bits ? int((1u << h->residual_shift) - 1u) : 0;
    if (scan_only) {  // every node is an "entry", read from the code array itself; the k best are the result
        a.entry = nullptr;
        a.entry_codes = h->d_codes.p;
        a.n_entry = uint32_t(h->n);
        a.n_seed = k;
    }
    CPB_CUDA(cudaMemsetAsync(a.next_query, 0, 4, st));
    // a narrow launch gives every query a block of its own (one warp or one team), so a handful of
    // queries spread over as many SMs and need as many visited slots
    const bool narrow = !cx.wide;
    const unsigned grid = narrow ? unsigned(nq) : unsigned(h->sm_count);
    const bool u16 = h->comp_bytes == 2;
    LaunchTimer timer(h, kKernelSearch, st);

    // two warps per query: asymmetric metric, table in shared memory, one adjacency row per warp
    // (beams over 1,024 up to 2,048 in its wide form, which exists for tables in shared memory; under the symmetric
    // metric only on packed sign bits, i.e. in binary-code mode)
    const bool team_ok = !scan_only && h->M <= 32 && h->k_entry <= 128 &&
                         (sym ? (a.packed != nullptr && beam <= 1024)
                              : ((beam <= 1024 || (beam <= 2048 && c.table_smem)) && (c.table_smem || h->K <= 32)));
    a.table_in_smem = c.table_smem ? 1 : 0;
    if (h->search_kernel == 2 && !team_ok && !sym) {
        set_error("search_kernel=2 needs the asymmetric metric, M <= 32, K*P*4 <= 32 KB or K <= 32, and a beam of at most 1024 (2048 with the table in shared memory)");
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    // (Also for a table too large for shared memory, read in place: on 1M x 960 clustered vectors the two-warp kernel
    // does 301 k queries/s against 237 k for one warp per query; only on vectors with independent coordinates, where an
    // expansion scores ~26 neighbours instead of ~2, one warp per query was 3-7 % ahead.)
    if (team_ok && h->search_kernel != 1) {
        const size_t per_team = (c.per_warp + search_team_extra_smem() + 15) & ~size_t(15);
        CPB_TRY(launch_search_team(h, a, per_team, narrow ? int(nq) : 0, st));
        h->launches++;
        CPB_CUDA(cudaGetLastError());
        return 0;
    }

#define CPB_SEARCH(U, T, S)                                                                                \
    do {                                                                                                   \
        cudaFuncAttributes fa;                                                                             \
        CPB_CUDA(cudaFuncGetAttributes(&fa, search_kernel<U, T, S>));                                      \
        int maxw = 65536 / (((fa.numRegs + 7) & ~7) * 32);                                                 \
        int w = narrow ? 1 : (c.warps < maxw ? c.warps : maxw);                                            \
        size_t smem = c.per_warp * w;                                                                      \
        CPB_CUDA(allow_max_dynamic_smem(search_kernel<U, T, S>));                                          \
        search_kernel<U, T, S><<<grid, w * 32, smem, st>>>(a);                                             \
    } while (0)
    if (sym && u16) CPB_SEARCH(true, false, true);
    else if (sym) CPB_SEARCH(false, false, true);
    else if (u16 && c.table_smem) CPB_SEARCH(true, true, false);
    else if (u16) CPB_SEARCH(true, false, false);
    else if (c.table_smem) CPB_SEARCH(false, true, false);
    else CPB_SEARCH(false, false, false);
#undef CPB_SEARCH
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace cpb
