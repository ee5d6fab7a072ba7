// Beam search with two warps per query ("team"): same algorithm and same results as
// search_kernel (search.cu), arranged so that every expansion is a short chain of instructions.
//
// The walker warp owns W and the visited marks and performs the expansions in the exact
// sequential order.  The scout warp prepares rows ahead of it.  Before each expansion the walker
// announces the node it expands and the next three unexpanded members of W.  During that
// expansion the scout prepares the first of them, the node the walker will select next unless
// this expansion admits something closer (about 3 % of the steps): it reads the visited bytes of
// the node's neighbours, scores the unvisited ones against the query table (which the two warps
// share in shared memory) and leaves ids, scores and a candidate mask in a result slot.  For the
// second announced node it loads the adjacency row, which it keeps in registers for its next
// turn, and asks for that row's visited bytes and codes to be brought into L2; the row of the third
// goes towards L2 as well.  When the walker selects a node that has a result slot, it drops the
// neighbours it has marked itself since the scout read the visited bytes (a ring of its latest
// marks tells which), marks the rest and admits them: no global load is left on its path.
// Without a slot it does the expansion itself, as the one-warp kernel does.  Scores are a pure
// function of (query, node) and the set of neighbours offered is the set unvisited at the
// walker's own sequential time either way, so the results do not depend on how far the scout got.
//
// W is a tiered vector: buckets of 32 slots, each a circular buffer, globally sorted.  An
// admission shifts inside one bucket (one load, two shuffles and one store per lane) and every
// later bucket takes the element pushed out of its predecessor at its front in place of its
// own last, all buckets at once (one lane per bucket).  While W still has room it is a plain array instead: every
// scored candidate is admitted then, so a row's candidates are appended, the closest unexpanded member is found by a
// scan, and the array is sorted once, when a row would overflow it or rows stop bringing more than a member or two.
//
// The two warps meet at a named barrier (bar.sync id, 64) once per expansion; every barrier sits
// in control flow that depends only on values both warps read after the previous barrier, so the
// two warps always execute the same sequence of barriers and nothing spins.  The entry scan and
// the rerank are split between the two warps.
//
// Used with M <= 32.  Asymmetric metric: the query table sits in shared memory when it is at most 32 KB and is read in
// place (global memory, through L1 / L2) otherwise; codes of up to 64 rotations are scored by the whole warp.
// Symmetric metric: binary-code mode only, on sign bits packed 32 per word (XOR and popcount, no table).  Beams up to
// 1,024 take 32 buckets, one per lane; beams up to 2,048 the wide form with 64 buckets, two per lane.
#include "search_common.cuh"

namespace cpb {
namespace {

using namespace srch;

constexpr int kSeedCap = 128;  // scout's seed list; the same arrays hold the result slots during the walk
constexpr int kSlots = 4;      // prepared rows kept for the walker (32 ids + 32 scores each)
constexpr int kRing = 64;      // ids the walker marked most recently
// mailbox words: 0 query, 8 scout evaluations, 9 scout seed count, 10 count; per result slot its
// node, candidate mask and the walker's mark count when the visited bytes were read; two
// announcement records {node, next three unexpanded, done, marks so far} used alternately
constexpr int kKeyBase = 16, kMaskBase = 20, kSnapBase = 24, kPostBase = 32;
constexpr int kMailWords = 48;
static_assert(kSlots * 32 <= kSeedCap, "result slots live in the seed arrays");

// ---- flat sorted list (the scout's share of the entry scan) ---------------------------------------
struct BeamList {
    float* d;
    uint32_t* id;
    uint32_t count, cap;
    float wd;
    uint32_t wi;
};

// Admission of (d, id), known to every lane, into a sorted list that keeps the cap best.
__device__ __forceinline__ void beam_admit(BeamList& L, float d, uint32_t id, int lane) {
    if (L.count == L.cap && !key_less(d, id, L.wd, L.wi)) return;
    uint32_t p = 0;
    if (L.count) {  // rank by a two-round 32-ary search
        const uint32_t stride = (L.count + 31) >> 5;
        const uint32_t e = min(L.count, (uint32_t(lane) + 1) * stride) - 1;
        const bool in = uint32_t(lane) * stride < L.count;
        const bool less = in && key_less(L.d[e], L.id[e], d, id);
        const uint32_t b = __popc(__ballot_sync(kFull, less));
        const uint32_t j = b * stride + lane;
        const bool less2 = b < 32 && uint32_t(lane) < stride && j < L.count && key_less(L.d[j], L.id[j], d, id);
        p = min(L.count, b * stride) + __popc(__ballot_sync(kFull, less2));
    }
    const int end = int(L.count == L.cap ? L.cap - 1 : L.count);
    for (int top = end; top > int(p); top -= 32) {
        const int i = top - 1 - lane;
        const bool act = i >= int(p);
        float md = 0.0f;
        uint32_t mi = 0;
        if (act) {
            md = L.d[i];
            mi = L.id[i];
        }
        __syncwarp();
        if (act) {
            L.d[i + 1] = md;
            L.id[i + 1] = mi;
        }
        __syncwarp();
    }
    if (lane == 0) {
        L.d[p] = d;
        L.id[p] = id;
    }
    __syncwarp();
    if (L.count < L.cap) ++L.count;
    if (L.count == L.cap) {
        L.wd = L.d[L.cap - 1];
        L.wi = L.id[L.cap - 1];
    }
}

__device__ __forceinline__ void beam_admit_lanes(BeamList& L, uint32_t m, bool mine, float dist, uint32_t id, int lane) {
    if (L.count == L.cap) m &= __ballot_sync(kFull, mine && key_less(dist, id, L.wd, L.wi));
    while (m) {
        const int src = __ffs(m) - 1;
        m &= m - 1;
        beam_admit(L, __shfl_sync(kFull, dist, src), __shfl_sync(kFull, id, src), lane);
    }
}

// ---- tiered sorted list (W, walker only) -----------------------------------------------------------
// Logical position p lives in bucket p >> 5 at slot (head + (p & 31)) & 31.  All nb * 32 logical
// positions always hold something: live members first (count of them), then members pushed out of
// a full list (still in ascending order, never looked at), then (+inf, invalid) fillers.  Lane b
// keeps bucket b's head and a copy of its last (largest) element.
struct TierList {
    float* d;
    uint32_t* id;    // expanded flag in the top bit
    int nb;          // buckets (cap / 32: up to 32, up to 64 in the wide form)
    uint32_t count, wcap, cur;
    float wd;        // worst live member once count == wcap
    uint32_t wi;
    int head;        // lane b: head of bucket b
    float max_d;     // lane b: last logical element of bucket b
    uint32_t max_i;
    int head2;       // wide form (beams over 1,024): lane b also keeps bucket 32 + b
    float max_d2;
    uint32_t max_i2;
};

// head of bucket b (b known to every lane)
template <bool WIDE>
__device__ __forceinline__ int tier_head(const TierList& T, int b) {
    if (WIDE && b >= 32) return __shfl_sync(kFull, T.head2, b - 32);
    return __shfl_sync(kFull, T.head, b);
}

// heads to zero (the arrays are then read flat) and the per-bucket maxima re-read
template <bool WIDE>
__device__ __forceinline__ void tier_reset_heads(TierList& T, int lane) {
    T.head = 0;
    T.max_d = INFINITY;
    T.max_i = kInvalidNode;
    if (lane < T.nb) {
        T.max_d = T.d[lane * 32 + 31];
        T.max_i = T.id[lane * 32 + 31];
    }
    if (WIDE) {
        T.head2 = 0;
        T.max_d2 = INFINITY;
        T.max_i2 = kInvalidNode;
        if (32 + lane < T.nb) {
            T.max_d2 = T.d[(32 + lane) * 32 + 31];
            T.max_i2 = T.id[(32 + lane) * 32 + 31];
        }
    }
}

template <bool WIDE>
__device__ __forceinline__ void tier_refresh_worst(TierList& T) {
    if (T.count == T.wcap) {
        const int wb = int(T.wcap - 1) >> 5;
        const int hw = tier_head<WIDE>(T, wb);
        const int ws = wb * 32 + ((hw + int((T.wcap - 1) & 31)) & 31);
        T.wd = T.d[ws];
        T.wi = T.id[ws] & kIdMask;
    }
}

// Admission of (d, id), known to every lane (search_engine.hpp:166-176).
template <bool WIDE>
__device__ __forceinline__ void tier_admit(TierList& T, float d, uint32_t id, int lane) {
    if (T.count == T.wcap && !key_less(d, id, T.wd, T.wi)) return;
    // first bucket whose largest element is not below the key (fillers are +inf: there is one); the maxima ascend
    // with the bucket, so the buckets below the key are a prefix and counting them gives the index
    const bool below = lane < T.nb && key_less(T.max_d, T.max_i & kIdMask, d, id);
    int b = __popc(__ballot_sync(kFull, below));
    if (WIDE) {
        const bool below2 = 32 + lane < T.nb && key_less(T.max_d2, T.max_i2 & kIdMask, d, id);
        b += __popc(__ballot_sync(kFull, below2));
    }
    const int hb = tier_head<WIDE>(T, b);
    const int slot = b * 32 + ((hb + lane) & 31);
    const float ed = T.d[slot];  // logical element `lane` of bucket b
    const uint32_t ei = T.id[slot];
    const int r = __popc(__ballot_sync(kFull, key_less(ed, ei & kIdMask, d, id)));  // rank inside the bucket (<= 31)
    const float pd = __shfl_up_sync(kFull, ed, 1);
    const uint32_t pi = __shfl_up_sync(kFull, ei, 1);
    const float nd = lane < r ? ed : (lane == r ? d : pd);
    const uint32_t ni = lane < r ? ei : (lane == r ? id : pi);
    if (lane >= r) {
        T.d[slot] = nd;
        T.id[slot] = ni;
    }
    const float out_d = __shfl_sync(kFull, ed, 31);  // pushed out of bucket b
    const uint32_t out_i = __shfl_sync(kFull, ei, 31);
    const float top_d = __shfl_sync(kFull, nd, 31);  // bucket b's new last element
    const uint32_t top_i = __shfl_sync(kFull, ni, 31);
    // later buckets, up to the one holding position wcap - 1: take the predecessor's last element
    // at the front, in the slot of the own last element, which moves on
    const int wb = int(T.wcap - 1) >> 5;
    const bool casc = lane > b && lane <= wb;
    const int last_slot = (lane & 31) * 32 + ((T.head + 31) & 31);
    float ld = out_d;
    uint32_t li = out_i;
    if (casc) {
        ld = T.d[last_slot];
        li = T.id[last_slot];
    }
    const float in_d = __shfl_up_sync(kFull, ld, 1);  // lane b passes on out_d
    const uint32_t in_i = __shfl_up_sync(kFull, li, 1);
    if (WIDE) {
        // the second set of buckets (32 + lane) does the same; bucket 32 takes what bucket 31 passes on
        const int bb = 32 + lane;
        const bool casc2 = bb > b && bb <= wb;
        const int last2 = bb * 32 + ((T.head2 + 31) & 31);
        float ld2 = out_d;
        uint32_t li2 = out_i;
        if (casc2) {
            ld2 = T.d[last2];
            li2 = T.id[last2];
        }
        float in2_d = __shfl_up_sync(kFull, ld2, 1);
        uint32_t in2_i = __shfl_up_sync(kFull, li2, 1);
        const float from31_d = __shfl_sync(kFull, ld, 31);
        const uint32_t from31_i = __shfl_sync(kFull, li, 31);
        if (lane == 0) {
            in2_d = from31_d;
            in2_i = from31_i;
        }
        if (casc2) {
            T.d[last2] = in2_d;
            T.id[last2] = in2_i;
            T.head2 = (T.head2 + 31) & 31;
            const int nl2 = bb * 32 + ((T.head2 + 31) & 31);
            T.max_d2 = T.d[nl2];
            T.max_i2 = T.id[nl2];
        }
        if (bb == b) {
            T.max_d2 = top_d;
            T.max_i2 = top_i;
        }
    }
    if (casc) {
        T.d[last_slot] = in_d;
        T.id[last_slot] = in_i;
        T.head = (T.head + 31) & 31;
        const int nl = lane * 32 + ((T.head + 31) & 31);
        T.max_d = T.d[nl];
        T.max_i = T.id[nl];
    }
    if (lane == b) {
        T.max_d = top_d;
        T.max_i = top_i;
    }
    __syncwarp();
    if (T.count < T.wcap) ++T.count;
    const uint32_t p = uint32_t(b) * 32 + r;
    if (p <= T.cur) T.cur = p;
    tier_refresh_worst<WIDE>(T);
}

// admit the scored candidates of the lanes in mask m, lowest lane first
template <bool WIDE>
__device__ __forceinline__ void tier_admit_lanes(TierList& T, uint32_t m, bool mine, float dist, uint32_t id, int lane) {
    if (T.count == T.wcap) m &= __ballot_sync(kFull, mine && key_less(dist, id, T.wd, T.wi));
    while (m) {
        const int src = __ffs(m) - 1;
        m &= m - 1;
        tier_admit<WIDE>(T, __shfl_sync(kFull, dist, src), __shfl_sync(kFull, id, src), lane);
    }
}

// ---- filling W (walker only) -----------------------------------------------------------------------
// Until W holds `wcap` members every scored candidate is admitted, so nothing has to be ranked: the walk
// starts with W as a plain array (live members in any order in [0, count), fillers behind), appends a row's
// candidates in one step and selects the closest unexpanded member by a scan.  The array is sorted once, when a
// row would overflow it, and the tiered list takes over.  The selected nodes and the final W are the same either
// way (the closest unexpanded member under the total order (distance, id); the wcap best of everything scored).
constexpr uint32_t kFillMin = 256;  // free places in W at the start of the walk from which the plain array pays (measured)

// bucket rotations undone: logical order becomes slot order (flags kept)
template <bool WIDE>
__device__ __forceinline__ void tier_flatten(TierList& T, int lane) {
    for (int b = 0; b < T.nb; ++b) {
        const int hb = tier_head<WIDE>(T, b);
        if (hb == 0) continue;
        const int from = b * 32 + ((hb + lane) & 31);
        const float v = T.d[from];
        const uint32_t w = T.id[from];
        __syncwarp();
        T.d[b * 32 + lane] = v;
        T.id[b * 32 + lane] = w;
    }
    __syncwarp();
    T.head = 0;
    if (WIDE) T.head2 = 0;
}

// the plain array becomes the tiered list: sorted, heads zero, cursor on the first unexpanded member
template <bool WIDE>
__device__ __forceinline__ void tier_from_plain(TierList& T, int lane) {
    int n = 32;
    while (n < int(T.count)) n <<= 1;
    __syncwarp();
    warp_sort_flagged(T.d, T.id, n, lane);
    tier_reset_heads<WIDE>(T, lane);
    T.cur = T.count;
    for (uint32_t base = 0; base < T.count; base += 32) {
        const uint32_t ei = T.id[base + lane];
        const uint32_t un = __ballot_sync(kFull, !(ei & kExpanded) && base + lane < T.count);
        if (un) {
            T.cur = base + uint32_t(__ffs(un) - 1);
            break;
        }
    }
    tier_refresh_worst<WIDE>(T);
}

// TSM: the query table is copied to shared memory (a compile-time fact, so that its reads stay
// shared-memory loads); otherwise it is read in place.
// No register cap: holding the kernel to 64 registers (15 teams per SM instead of 11 when the table is read in
// place) spills inside the walk and was measured slower on every configuration.
template <bool U16, bool TSM, bool K2, bool WIDE, bool SYM>
__global__ void search_team_kernel(SearchArgs a) {
    extern __shared__ __align__(16) unsigned char team_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int team = warp >> 1, role = warp & 1, teams = blockDim.x >> 6;
    const int tl = role * 32 + lane;  // 0..63 within the team
    const size_t table_floats = size_t(a.K) * a.P;
    const size_t dim_pad = a.qsm_floats;
    const int cap = int(a.cap);
    unsigned char* mine = team_smem + size_t(a.per_warp_smem) * team;  // per-team area
    float* table_sm = reinterpret_cast<float*>(mine);  // the query table, when it fits
    float* qsm = table_sm + (TSM ? table_floats : 0);
    uint32_t* sid = reinterpret_cast<uint32_t*>(qsm + dim_pad);
    float* sd = reinterpret_cast<float*>(sid + cap);
    uint32_t* seed_id = reinterpret_cast<uint32_t*>(sd + cap);  // scout's seeds
    float* seed_d = reinterpret_cast<float*>(seed_id + kSeedCap);
    uint32_t* res_id = seed_id;  // [kSlots][32] rows prepared by the scout (after the entry scan)
    float* res_d = seed_d;       // [kSlots][32]
    uint32_t* ring = reinterpret_cast<uint32_t*>(seed_d + kSeedCap);
    volatile uint32_t* mail = reinterpret_cast<volatile uint32_t*>(ring + kRing);

    auto team_sync = [&]() {
        __syncwarp();
        asm volatile("bar.sync %0, 64;" ::"r"(team + 1) : "memory");
    };

    const uint32_t slot = blockIdx.x * teams + team;
    uint8_t* vis = a.visited + size_t(slot) * a.vis_stride;
    uint32_t epoch = a.epochs[slot];
    const uint32_t beam = a.beam;
    const bool scan_mode = a.n_seed < a.n_entry;
    const int row_bytes = a.K * (U16 ? 2 : 1);
    const bool coop_ok = !SYM && a.K <= 64;
    // symmetric metric (binary-code mode): the query's code follows its vector in the team's query area, its packed sign
    // bits follow the code; the walk compares packed bits, the entry scan the contiguous byte copy of the entry codes
    const unsigned char* qcode_sm = reinterpret_cast<const unsigned char*>(qsm + a.qvec_floats);
    uint32_t* qpacked_sm = reinterpret_cast<uint32_t*>(qsm + a.qvec_floats + ((row_bytes + 15) / 16) * 4);
    constexpr bool two_blocks = K2;  // 32 < K <= 64: a lane owns two rotations in the whole-warp scoring (a compile-time
                                     // fact, so that the narrower codes pay nothing for it)

    while (true) {
        if (role == 0 && lane == 0) mail[0] = atomicAdd(a.next_query, 1u);
        team_sync();
        const uint32_t q = mail[0];
        if (q >= a.nq) break;
        // a table too large for shared memory is read in place (through L1 / L2)
        const float* table = SYM ? nullptr : (TSM ? table_sm : a.tables + size_t(q) * table_floats);
        // one lane scores one node (row `row` of `code_base`) under the kernel's metric
        auto score_lane = [&](const void* code_base, uint32_t row) -> float {
            if (SYM) {
                if (code_base == a.codes) return packed_distance_lane(qpacked_sm, a.packed, row, a.packed_words, a.resid_kp, a.resid_mul);
                return sym_distance_lane<U16>(qcode_sm, code_base, row, a.K, a.resid_kp, a.resid_mul);
            }
            return asym_distance_lane<U16>(table, code_base, row, a.K, a.P);
        };
        {   // set-up by all 64 lanes
            if (TSM) {
                const float4* src = reinterpret_cast<const float4*>(a.tables + size_t(q) * table_floats);
                float4* dst = reinterpret_cast<float4*>(table_sm);
                for (int i = tl; i < int(table_floats / 4); i += 64) dst[i] = __ldg(src + i);
            }
            if (a.rerank_k) {
                const float* qv = a.queries + size_t(q) * a.dim;
                for (int i = tl; i < int(SYM ? a.qvec_floats : dim_pad); i += 64) qsm[i] = i < a.dim ? __ldg(qv + i) : 0.0f;
            }
            if (SYM) {
                const unsigned char* src = static_cast<const unsigned char*>(a.qcodes) + size_t(q) * row_bytes;
                for (int i = tl; i < row_bytes; i += 64) reinterpret_cast<unsigned char*>(qsm + a.qvec_floats)[i] = src[i];
                if (role == 0) {  // the packed bits straight from the code in global memory (one warp: the vote is its own)
                    for (int w = 0; w < a.packed_words; ++w) {
                        const int r = 32 * w + lane;
                        const uint32_t word = __ballot_sync(kFull, r < a.K && (src[r * (U16 ? 2 : 1)] & 1u));
                        if (lane == 0) qpacked_sm[w] = word;
                    }
                }
            }
            for (int p = tl; p < cap; p += 64) {
                sd[p] = INFINITY;
                sid[p] = kInvalidNode;
            }
            if (++epoch == 256) {  // the 8-bit epoch wraps: forget every earlier query
                uint4* v4 = reinterpret_cast<uint4*>(vis);
                for (uint64_t i = tl; i < a.vis_stride / 16; i += 64) v4[i] = make_uint4(0u, 0u, 0u, 0u);
                epoch = 1;
            }
            if (tl < kSlots) mail[kKeyBase + tl] = kInvalidNode;
        }
        team_sync();

        uint32_t nexp = 0, nevals = 0;
        TierList T;  // the walker's W
        T.d = sd;
        T.id = sid;
        T.nb = cap >> 5;
        T.count = 0;
        T.cur = 0;
        T.wcap = scan_mode ? a.n_seed : beam;
        T.wd = INFINITY;
        T.wi = kInvalidNode;
        T.head = 0;
        T.max_d = INFINITY;
        T.max_i = kInvalidNode;
        T.head2 = 0;
        T.max_d2 = INFINITY;
        T.max_i2 = kInvalidNode;
        uint32_t total_marks = 0;  // walker: nodes marked since the query began (ring write position)

        // admissions go to the plain array while W is filling, to the tiered list afterwards
        bool filling = false;
        auto admit_one = [&](float d, uint32_t id) {  // (d, id) known to every lane
            if (filling) {
                if (T.count < T.wcap) {
                    if (lane == 0) {
                        sd[T.count] = d;
                        sid[T.count] = id;
                    }
                    ++T.count;
                    __syncwarp();
                    return;
                }
                tier_from_plain<WIDE>(T, lane);
                filling = false;
            }
            tier_admit<WIDE>(T, d, id, lane);
        };
        auto admit_lanes = [&](uint32_t m, bool mine, float dist, uint32_t id) {
            if (filling) {
                const uint32_t nf = uint32_t(__popc(m));
                if (T.count + nf <= T.wcap) {
                    if (mine) {
                        const uint32_t pos = T.count + uint32_t(__popc(m & ((1u << lane) - 1u)));
                        sd[pos] = dist;
                        sid[pos] = id;
                    }
                    T.count += nf;
                    __syncwarp();
                    return;
                }
                tier_from_plain<WIDE>(T, lane);
                filling = false;
            }
            tier_admit_lanes<WIDE>(T, m, mine, dist, id, lane);
        };

        // walker alone: visited test-and-set of one row, scoring, admission
        // (search_engine.hpp:153-177); the marked ids go to the ring
        auto offer = [&](uint32_t id, bool in_range) {
            bool fresh = in_range;
            if (!a.rows_distinct) {  // every lane takes part in the match, in range or not
                const uint32_t grp = __match_any_sync(kFull, id);
                fresh = fresh && (__ffs(grp) - 1) == lane;
            }
            if (fresh) {
                if (__ldcg(vis + id) == epoch) fresh = false;
                else vis[id] = uint8_t(epoch);
            }
            uint32_t m = __ballot_sync(kFull, fresh);
            if (fresh) ring[(total_marks + __popc(m & ((1u << lane) - 1u))) & (kRing - 1)] = id;
            const int nf = __popc(m);
            total_marks += nf;
            nevals += nf;
            if (nf == 0) return;
            if (coop_ok && nf <= kCoopMax) {
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
                        if (two_blocks && 32 + lane < a.K) comph[f] = load_component<U16>(crow, 32 + lane);
                    }
                }
#pragma unroll
                for (int f = 0; f < kCoopMax; ++f)
                    if (f < nf)
                        admit_one(two_blocks ? asym_distance_coop2(table, a.K, a.P, comp[f], comph[f], lane)
                                             : asym_distance_coop(table, a.K, a.P, comp[f], lane), cid[f]);
            } else {
                float dist = 0.0f;
                if (fresh) dist = score_lane(a.codes, id);
                admit_lanes(m, fresh, dist, id);
            }
        };

        if (scan_mode) {
            // entry scan: the two warps take alternate batches and keep their own n_seed best
            BeamList S;  // the scout's
            S.d = seed_d;
            S.id = seed_id;
            S.count = 0;
            S.cap = a.n_seed;
            S.wd = INFINITY;
            S.wi = kInvalidNode;
            for (uint32_t e0 = 32u * role; e0 < a.n_entry; e0 += 64) {
                const uint32_t e = e0 + lane;
                if (e + 64 < a.n_entry) {
                    prefetch_l1(a.entry + e + 64);
                    prefetch_l1(static_cast<const unsigned char*>(a.entry_codes) + size_t(e + 64) * row_bytes);
                }
                const uint32_t id = e < a.n_entry ? __ldg(a.entry + e) : kInvalidNode;
                const bool ok = id < a.n;
                float dist = 0.0f;
                if (ok) dist = score_lane(a.entry_codes, e);
                const uint32_t m = __ballot_sync(kFull, ok);
                nevals += __popc(m);
                if (role == 0) tier_admit_lanes<WIDE>(T, m, ok, dist, id, lane);
                else beam_admit_lanes(S, m, ok, dist, id, lane);
            }
            if (role == 1 && lane == 0) {
                mail[8] = nevals;
                mail[9] = S.count;
            }
            team_sync();
            if (role == 0) {
                const uint32_t n1 = mail[9];
                nevals += mail[8];
                for (uint32_t i = 0; i < n1; ++i) tier_admit<WIDE>(T, seed_d[i], seed_id[i], lane);
                // W now holds the seeds (within bucket (n_seed - 1) / 32 and before): bring it back
                // to a flat list, fillers after the live members
                const int wb = int(T.wcap - 1) >> 5;
                for (int b = 0; b <= wb; ++b) {
                    const int hb = tier_head<WIDE>(T, b);
                    const int from = b * 32 + ((hb + lane) & 31);
                    float v = sd[from];
                    uint32_t w = sid[from];
                    if (uint32_t(b * 32 + lane) >= T.count) {
                        v = INFINITY;
                        w = kInvalidNode;
                    }
                    __syncwarp();
                    sd[b * 32 + lane] = v;
                    sid[b * 32 + lane] = w;
                }
                __syncwarp();
                // the seeds are offered to the walk: mark them visited
                const uint32_t nseeds = T.count;
                nevals += nseeds;
                for (uint32_t p = lane; p < nseeds; p += 32) vis[sid[p]] = uint8_t(epoch);
                if (nseeds > beam) {  // a beam narrower than the seed set keeps the best `beam` seeds
                    __syncwarp();
                    for (uint32_t p = beam + lane; p < uint32_t(wb + 1) * 32; p += 32) {
                        sd[p] = INFINITY;
                        sid[p] = kInvalidNode;
                    }
                    T.count = beam;
                }
                __syncwarp();
                T.wcap = beam;
                T.cur = 0;
                tier_reset_heads<WIDE>(T, lane);
                tier_refresh_worst<WIDE>(T);
            }
        } else if (role == 0) {
            for (uint32_t e0 = 0; e0 < a.n_entry; e0 += 32) {  // search_engine.hpp:105-115
                const uint32_t e = e0 + lane;
                const uint32_t id = e < a.n_entry ? __ldg(a.entry + e) : kInvalidNode;
                offer(id, id < a.n);
            }
        }

        // ---- walk
        // Walker and scout meet at one barrier per expansion.  Before the barrier the walker selects
        // the node to expand and announces it together with the next three unexpanded members of W;
        // after it the walker consumes the prepared row of that node (if the scout has one) while the
        // scout moves the announced nodes one stage further.
        if (role == 0 && T.wcap >= T.count + kFillMin) {
            tier_flatten<WIDE>(T, lane);
            filling = true;
        }
        uint32_t low_rows = 0;  // walker: consecutive expansions that brought at most two new members
        uint32_t rkey = kInvalidNode;  // scout: lane j < kSlots holds the node of result slot j
        uint32_t held_key = kInvalidNode, held_id = kInvalidNode;  // scout: adjacency row loaded at the previous turn
        uint32_t step = 0;
        while (true) {
            volatile uint32_t* mb = mail + kPostBase + (step & 1) * 8;  // this step's announcement
            if (role == 0 && filling) {
                // the two closest unexpanded members of the plain array: the first is expanded now, the second announced
                float b1d = INFINITY, b2d = INFINITY;
                uint32_t b1i = kInvalidNode, b2i = kInvalidNode;
                int b1s = 0;
                for (uint32_t p = lane; p < T.count; p += 32) {
                    const float v = sd[p];
                    const uint32_t w = sid[p];
                    if (!(w & kExpanded)) {
                        if (key_less(v, w, b1d, b1i)) {
                            b2d = b1d;
                            b2i = b1i;
                            b1d = v;
                            b1i = w;
                            b1s = int(p);
                        } else if (key_less(v, w, b2d, b2i)) {
                            b2d = v;
                            b2i = w;
                        }
                    }
                }
                float md = b1d;
                uint32_t mi = b1i;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) {
                    const float od = __shfl_xor_sync(kFull, md, o);
                    const uint32_t oi = __shfl_xor_sync(kFull, mi, o);
                    if (key_less(od, oi, md, mi)) {
                        md = od;
                        mi = oi;
                    }
                }
                if (mi != kInvalidNode) {
                    const bool win = b1i == mi;  // ids are unique in W
                    if (win) sid[b1s] = mi | kExpanded;
                    ++nexp;
                    float xd = win ? b2d : b1d;
                    uint32_t xi = win ? b2i : b1i;
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) {
                        const float od = __shfl_xor_sync(kFull, xd, o);
                        const uint32_t oi = __shfl_xor_sync(kFull, xi, o);
                        if (key_less(od, oi, xd, xi)) {
                            xd = od;
                            xi = oi;
                        }
                    }
                    if (lane == 0) {
                        mb[0] = mi;
                        mb[1] = xi;
                        mb[2] = kInvalidNode;
                        mb[3] = kInvalidNode;
                        mb[4] = 0;
                        mb[5] = total_marks;
                    }
                    __syncwarp();
                } else if (lane == 0) {
                    mb[4] = 1;
                }
            } else if (role == 0) {
                if (T.cur < T.count) {
                    // closest member of W that has not been expanded (search_engine.hpp:121-123)
                    const int cb = int(T.cur >> 5), cl = int(T.cur & 31);
                    const int hb = tier_head<WIDE>(T, cb);
                    const int cslot = cb * 32 + ((hb + lane) & 31);
                    uint32_t ei = sid[cslot];  // logical element `lane` of the cursor's bucket
                    const uint32_t node = __shfl_sync(kFull, ei, cl) & kIdMask;
                    if (lane == cl) sid[cslot] = ei | kExpanded;
                    ++nexp;
                    // the next unexpanded members: the first is the new cursor
                    uint32_t base = uint32_t(cb) * 32;
                    uint32_t un = __ballot_sync(kFull, !(ei & kExpanded) && lane > cl && base + lane < T.count);
                    while (!un) {
                        base += 32;
                        if (base >= T.count) break;
                        const int h2 = tier_head<WIDE>(T, int(base >> 5));
                        ei = sid[base + ((h2 + lane) & 31)];
                        un = __ballot_sync(kFull, !(ei & kExpanded) && base + lane < T.count);
                    }
                    uint32_t p0 = kInvalidNode, p1 = kInvalidNode, p2 = kInvalidNode;
                    T.cur = T.count;
                    if (un) {
                        int b = __ffs(un) - 1;
                        T.cur = base + b;
                        p0 = __shfl_sync(kFull, ei, b);
                        un &= un - 1;
                        if (un) {
                            b = __ffs(un) - 1;
                            p1 = __shfl_sync(kFull, ei, b);
                            un &= un - 1;
                            if (un) p2 = __shfl_sync(kFull, ei, __ffs(un) - 1);
                        }
                    }
                    if (lane == 0) {
                        mb[0] = node;
                        mb[1] = p0;
                        mb[2] = p1;
                        mb[3] = p2;
                        mb[4] = 0;
                        mb[5] = total_marks;
                    }
                } else if (lane == 0) {
                    mb[4] = 1;
                }
            }
            team_sync();
            if (mb[4]) break;
            const uint32_t node = mb[0];
            if (role == 0) {
                const uint32_t evals_before = nevals;
                // result slot of this node, if the scout got that far
                uint32_t key = kInvalidNode;
                if (lane < kSlots) key = mail[kKeyBase + lane];
                const uint32_t match = __ballot_sync(kFull, key == node);
                int s = match ? __ffs(match) - 1 : -1;
                uint32_t snap = 0;
                if (s >= 0) {
                    snap = mail[kSnapBase + s];
                    if (total_marks - snap > 32) s = -1;  // too many marks since the scout looked: do it here
                }
                if (s >= 0) {
                    const uint32_t id = res_id[s * 32 + lane];
                    const float dist = res_d[s * 32 + lane];
                    bool fresh = (mail[kMaskBase + s] >> lane) & 1u;
                    // neighbours marked since the scout read the visited bytes are no longer fresh
                    const uint32_t cnt = total_marks - snap;
                    const uint32_t rv = uint32_t(lane) < cnt ? ring[(snap + lane) & (kRing - 1)] : kInvalidNode;
                    for (uint32_t j = 0; j < cnt; ++j)
                        if (__shfl_sync(kFull, rv, int(j)) == id) fresh = false;
                    if (fresh) vis[id] = uint8_t(epoch);
                    const uint32_t fm = __ballot_sync(kFull, fresh);
                    if (fresh) ring[(total_marks + __popc(fm & ((1u << lane) - 1u))) & (kRing - 1)] = id;
                    total_marks += __popc(fm);
                    nevals += __popc(fm);
                    admit_lanes(fm, fresh, dist, id);
                } else {
                    const uint32_t id = lane < a.M ? __ldg(a.adj + size_t(node) * a.M + lane) : kInvalidNode;
                    offer(id, id < a.n);
                }
                // the plain array is left as soon as it stops paying: once rows bring a member or two, ranking them
                // costs less than scanning the array at every selection
                if (filling) {
                    low_rows = nevals - evals_before <= 2 ? low_rows + 1 : 0;
                    if (low_rows >= 3) {
                        tier_from_plain<WIDE>(T, lane);
                        filling = false;
                    }
                }
            } else {
                // The load the turn waits for goes out first: the visited bytes of the neighbours of P0, the node
                // selected next (its row is normally in registers since the last turn).  Whether the row is already
                // prepared is only known a few instructions later; the bytes are asked for either way.
                const uint32_t P0 = mb[1];
                uint32_t u_id = kInvalidNode;
                if (P0 != kInvalidNode) {
                    if (held_key == P0) u_id = held_id;
                    else if (lane < a.M) u_id = __ldg(a.adj + size_t(P0) * a.M + lane);
                }
                bool u_first = u_id < a.n;
                if (!a.rows_distinct) {
                    const uint32_t grp = __match_any_sync(kFull, u_id);
                    u_first = u_first && (__ffs(grp) - 1) == lane;
                }
                uint32_t u_vis = 0;
                if (u_first) u_vis = __ldcg(vis + u_id);
                const uint32_t P1 = mb[2], P2 = mb[3], snap = mb[5];
                // adjacency row of the node three expansions away towards L2
                if (lane == 0 && P2 != kInvalidNode) {
                    prefetch_l2(a.adj + size_t(P2) * a.M);
                    prefetch_l2(a.adj + size_t(P2) * a.M + a.M - 1);
                }
                auto in_r = [&](uint32_t x) { return __ballot_sync(kFull, rkey == x) != 0u; };
                const bool do_u = P0 != kInvalidNode && !in_r(P0);  // the node selected next: prepare it now
                const bool do_v = P1 != kInvalidNode && !in_r(P1);  // the one after: bring its data closer
                // the row of P1 is loaded now and kept for the next turn, when P1 has become P0
                uint32_t v_id = kInvalidNode;
                if (do_v) {
                    if (held_key == P1) v_id = held_id;
                    else if (lane < a.M) v_id = __ldg(a.adj + size_t(P1) * a.M + lane);
                }
                if (do_u) {
                    // a slot whose node is neither being consumed nor announced
                    const bool keep = rkey != kInvalidNode && (rkey == node || rkey == P0 || rkey == P1 || rkey == P2);
                    const uint32_t free_slots = __ballot_sync(kFull, lane < kSlots && !keep);
                    const int s = __ffs(free_slots) - 1;  // at most three of the four are kept
                    const bool cand = u_first && u_vis != epoch;
                    const uint32_t u_mask = __ballot_sync(kFull, cand);
                    const int nf = __popc(u_mask);
                    float dist = 0.0f;
                    if (coop_ok && nf <= kCoopMax) {
                        uint32_t m = u_mask;
                        for (int f = 0; f < nf; f += 2) {  // two candidates per round
                            const int s0 = __ffs(m) - 1;
                            m &= m - 1;
                            const int s1 = m ? __ffs(m) - 1 : s0;
                            m &= m - 1;
                            const uint32_t id0 = __shfl_sync(kFull, u_id, s0), id1 = __shfl_sync(kFull, u_id, s1);
                            uint32_t comp0 = 0, comp1 = 0, comp0h = 0, comp1h = 0;
                            const unsigned char* row0 = static_cast<const unsigned char*>(a.codes) + size_t(id0) * row_bytes;
                            const unsigned char* row1 = static_cast<const unsigned char*>(a.codes) + size_t(id1) * row_bytes;
                            if (lane < a.K) {
                                comp0 = load_component<U16>(row0, lane);
                                comp1 = load_component<U16>(row1, lane);
                            }
                            if (two_blocks && 32 + lane < a.K) {
                                comp0h = load_component<U16>(row0, 32 + lane);
                                comp1h = load_component<U16>(row1, 32 + lane);
                            }
                            const float d0 = two_blocks ? asym_distance_coop2(table, a.K, a.P, comp0, comp0h, lane)
                                                        : asym_distance_coop(table, a.K, a.P, comp0, lane);
                            const float d1 = two_blocks ? asym_distance_coop2(table, a.K, a.P, comp1, comp1h, lane)
                                                        : asym_distance_coop(table, a.K, a.P, comp1, lane);
                            if (lane == s0) dist = d0;
                            if (lane == s1) dist = d1;
                        }
                    } else if (cand) {
                        dist = score_lane(a.codes, u_id);
                    }
                    if (s >= 0) {
                        res_id[s * 32 + lane] = u_id;
                        res_d[s * 32 + lane] = dist;
                        if (lane == 0) {
                            mail[kMaskBase + s] = u_mask;
                            mail[kSnapBase + s] = snap;
                            mail[kKeyBase + s] = P0;
                        }
                        if (lane == s) rkey = P0;
                    }
                }
                if (do_v) {  // visited bytes and codes of the next row towards L2
                    if (v_id < a.n && held_key != P1) {
                        prefetch_l2(vis + v_id);
                        if (SYM) prefetch_l2(a.packed + size_t(v_id) * a.packed_words);  // (the byte codes are not resident)
                        else prefetch_l2(static_cast<const unsigned char*>(a.codes) + size_t(v_id) * row_bytes);
                    }
                    held_key = P1;
                    held_id = v_id;
                }
            }
            ++step;
        }

        // ---- rerank (both warps) and output (walker)
        if (role == 0) {
            if (filling) tier_from_plain<WIDE>(T, lane);  // W never filled: sorted now
            // back to a flat list, expanded flags dropped
            const int nbl = int(T.count + 31) >> 5;
            for (int b = 0; b < nbl; ++b) {
                const int hb = tier_head<WIDE>(T, b);
                const int from = b * 32 + ((hb + lane) & 31);
                const float v = sd[from];
                const uint32_t w = sid[from];
                __syncwarp();
                sd[b * 32 + lane] = v;
                sid[b * 32 + lane] = uint32_t(b * 32 + lane) < T.count ? (w & kIdMask) : kInvalidNode;
            }
            if (lane == 0) mail[10] = T.count;
        }
        team_sync();
        const uint32_t count = mail[10];
        int nsort = 32;
        while (nsort < int(count)) nsort <<= 1;
        uint32_t ncand = 0;
        if (a.rerank_k) {
            ncand = min(a.rerank_k, count);
            const int g = lane >> 3, j = lane & 7;
            const bool vec4 = (a.dim & 3) == 0;
#pragma unroll 2
            for (uint32_t c0 = 4u * role; c0 < ncand; c0 += 8) {
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
        }
        team_sync();
        if (role == 0) {
            if (a.rerank_k) {
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
        }
        // the barrier at the top of the loop keeps the scout off the shared arrays until the
        // walker is done with them
    }
    if (role == 0 && lane == 0) a.epochs[slot] = epoch;
}

}  // namespace

// bytes of shared memory one team needs on top of the query table
size_t search_team_extra_smem() { return size_t(kSeedCap) * 8 + kRing * 4 + kMailWords * 4; }

// Teams per block: as many as shared memory allows (at most 15, one named barrier each), fewer if
// the register file does not hold them.
template <bool U16, bool TSM, bool K2, bool WIDE, bool SYM>
static int launch_team_t(cphnsw_b200_index* h, SearchArgs a, size_t per_team, int narrow_blocks, cudaStream_t st) {
    auto kernel = search_team_kernel<U16, TSM, K2, WIDE, SYM>;
    int teams = int((226 * 1024) / per_team);
    if (teams > 15) teams = 15;
    if (narrow_blocks) teams = 1;  // one query per block
    for (; teams >= 1; --teams) {
        int blocks = 0;
        CPB_CUDA(allow_max_dynamic_smem(kernel));
        CPB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, teams * 64, per_team * teams));
        if (blocks >= 1) break;
    }
    if (teams < 1) {
        set_error("search: no launch configuration fits the two-warp kernel");
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    kernel<<<narrow_blocks ? unsigned(narrow_blocks) : unsigned(h->sm_count), teams * 64, per_team * teams, st>>>(a);
    return 0;
}

int launch_search_team(cphnsw_b200_index* h, SearchArgs a, size_t per_team, int narrow_blocks, cudaStream_t st) {
    a.per_warp_smem = uint32_t(per_team);
    const bool u16 = h->comp_bytes == 2, k2 = h->K > 32, wide = a.cap > 1024;
#define CPB_TEAM(U, T, W, X) launch_team_t<U, T, W, X, false>(h, a, per_team, narrow_blocks, st)
    // binary-code mode: symmetric metric on packed sign bits, no query table
    if (a.packed) return u16 ? launch_team_t<true, false, false, false, true>(h, a, per_team, narrow_blocks, st)
                             : launch_team_t<false, false, false, false, true>(h, a, per_team, narrow_blocks, st);
    if (a.table_in_smem) {
        if (wide) {  // beams over 1,024: 64 buckets, two per lane
            if (k2) return u16 ? CPB_TEAM(true, true, true, true) : CPB_TEAM(false, true, true, true);
            return u16 ? CPB_TEAM(true, true, false, true) : CPB_TEAM(false, true, false, true);
        }
        if (k2) return u16 ? CPB_TEAM(true, true, true, false) : CPB_TEAM(false, true, true, false);
        return u16 ? CPB_TEAM(true, true, false, false) : CPB_TEAM(false, true, false, false);
    }
    // a table read in place belongs to K <= 32 and beams up to 1,024 here
    return u16 ? CPB_TEAM(true, false, false, false) : CPB_TEAM(false, false, false, false);
#undef CPB_TEAM
}

}  // namespace cpb
