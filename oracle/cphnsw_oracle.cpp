// CPU oracle for the CP-HNSW hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, on the CPU and in the plainest possible form, the arithmetic
// of the reference project's encode -> code distance -> kNN graph -> select_neighbors
// -> beam search -> rerank path.  It exists so that the CUDA library can be checked
// against it; nothing in the product links, loads or calls it.  Only the test-suite,
// the smoke check and the CPU-baseline leg of the benchmark may load this library.
//
// Parity status: the FHT, the sign tables, the rotation and the K-byte code are pinned
// against the reference's own headers compiled in place (see ref_shim.cpp and the golden
// fixtures).  Code distance, kNN lists, select_neighbors, beam search, rerank and
// multiprobe follow call sites and papers only, because the reference's legacy sources
// for them are absent from its tree: for those functions parity is UNPINNED by any
// reference-side golden vector.
//
// Every function cites the reference file:line it follows (paths relative to the
// reference project root).
//
// Build: g++ -O2 -fopenmp -ffp-contract=off -shared -fPIC (see Makefile).  Contraction is
// off so that every float add below is a single IEEE operation in program order.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <queue>
#include <random>
#include <set>
#include <utility>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(CPHNSW_ORACLE_TUNED) && defined(__AVX512F__)
#include <immintrin.h>
#endif

namespace {

constexpr uint32_t kInvalid = 0xFFFFFFFFu;  // include/cphnsw/core/types.hpp:28-30 (INVALID_NODE)

size_t next_pow2(size_t n) {  // include/cphnsw/encoder/rotation.hpp:128-132
    size_t p = 1;
    while (p < n) p *= 2;
    return p;
}

// include/cphnsw/encoder/transform/fht.hpp:56-69 (fht_scalar): stages h = 1, 2, 4, ...;
// each butterfly writes lo = x + y, hi = x - y.
void fht_scalar(float* v, size_t n) {
    for (size_t h = 1; h < n; h *= 2)
        for (size_t i = 0; i < n; i += 2 * h)
            for (size_t j = i; j < i + h; ++j) {
                float x = v[j], y = v[j + h];
                v[j] = x + y;
                v[j + h] = x - y;
            }
}

// Width of the in-register phase the reference's SIMD FHT runs for a given build and length.
// fht.hpp:141-147: the AVX-512 routine defers to AVX2 below 16; fht.hpp:81-87: AVX2 defers
// to scalar below 8.  convention: 0 scalar build, 1 AVX2 build, 2 AVX-512 build.
size_t simd_width(int convention, size_t n) {
    if (convention == 2 && n >= 16) return 16;
    if (convention >= 1 && n >= 8) return 8;
    return 1;
}

// The reference's SIMD FHT.  Its in-register stages (fht.hpp:96-111 for AVX2, :155-180 for
// AVX-512) blend `v - v_swap` into the upper lane of each pair, i.e. hi = y - x, where the
// scalar butterfly writes x - y.  Every later stage only adds or subtracts whole values, so
// the result equals the scalar transform with element i negated when popcount(i & (W-1))
// is odd; magnitudes are bit-equal.
void fht_convention(float* v, size_t n, int convention) {
    fht_scalar(v, n);
    size_t w = simd_width(convention, n);
    if (w > 1)
        for (size_t i = 0; i < n; ++i)
            if (__builtin_popcountll(i & (w - 1)) & 1) v[i] = -v[i];
}

// include/cphnsw/encoder/rotation.hpp:90-111 (apply_copy + apply): zero-pad, then three times
// (multiply by the +-1 diagonal, FHT).
void rotate(const float* x, size_t dim, size_t P, const int8_t* signs /*[3][P]*/, int convention,
            float* buf) {
    std::memcpy(buf, x, dim * sizeof(float));
    std::memset(buf + dim, 0, (P - dim) * sizeof(float));
    for (int layer = 0; layer < 3; ++layer) {
        const int8_t* s = signs + (size_t)layer * P;
        for (size_t i = 0; i < P; ++i) buf[i] *= static_cast<float>(s[i]);  // rotation.hpp:146-150
        fht_convention(buf, P, convention);
    }
}

// include/cphnsw/encoder/cp_encoder.hpp:78-91 (scalar form; the AVX-512 form at :27-76 returns
// the same index: first position whose magnitude equals the maximum).
void argmax_abs(const float* b, size_t n, size_t& idx, float& mag) {
    idx = 0;
    mag = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float a = std::fabs(b[i]);
        if (a > mag) {
            mag = a;
            idx = i;
        }
    }
}

// include/cphnsw/core/types.hpp:88-90 (CPCode::encode): component = (index << 1) | negative.
inline uint32_t component(size_t idx, bool neg) { return (uint32_t)((idx << 1) | (neg ? 1 : 0)); }

inline uint32_t load_comp(const void* codes, size_t comp_bytes, size_t i) {
    return comp_bytes == 1 ? ((const uint8_t*)codes)[i] : ((const uint16_t*)codes)[i];
}
inline void store_comp(void* codes, size_t comp_bytes, size_t i, uint32_t c) {
    if (comp_bytes == 1)
        ((uint8_t*)codes)[i] = (uint8_t)c;
    else
        ((uint16_t*)codes)[i] = (uint16_t)c;
}

// Legacy hamming_distance(CPCode, CPCode): number of the K components that differ
// (use sites: evaluation/debug_estimator.cpp:149,172; evaluation/debug_code_storage.cpp:81).
// Residual codes of the unified index (include/cphnsw/core/types.hpp:284-302;
// hamming_combined_scalar, include/cphnsw/distance/detail/scalar_kernels.hpp:57-76): with the first
// g_primary components the primary bits and the others the residual bits, the distance is
// (h_primary << g_shift) + h_residual.  g_primary = 0 (the default) is the plain count.  A setting
// of the whole oracle (orc_set_residual_weighting), so that every function built on code_dist follows it.
static size_t g_primary = 0;
static uint32_t g_shift = 0;
inline uint32_t code_dist(const void* a, size_t ia, const void* b, size_t ib, size_t K,
                          size_t comp_bytes) {
#ifdef CPHNSW_ORACLE_TUNED
    // the tuned build (CPU baseline of the benchmark): byte codes of whole 8-byte words without residual
    // weighting are compared a word at a time - 32 bytes at a time where the host has AVX-512BW/VL
    if (comp_bytes == 1 && g_primary == 0 && (K & 7) == 0) {
        const uint8_t* pa = (const uint8_t*)a + ia * K;
        const uint8_t* pb = (const uint8_t*)b + ib * K;
        uint32_t dd = 0;
        size_t r = 0;
#if defined(__AVX512BW__) && defined(__AVX512VL__)
        for (; r + 32 <= K; r += 32)
            dd += (uint32_t)__builtin_popcount(_mm256_cmpneq_epi8_mask(_mm256_loadu_si256((const __m256i*)(pa + r)),
                                                                       _mm256_loadu_si256((const __m256i*)(pb + r))));
#endif
        for (; r < K; r += 8) {
            uint64_t x, y;
            std::memcpy(&x, pa + r, 8);
            std::memcpy(&y, pb + r, 8);
            x ^= y;
            const uint64_t lo = 0x7f7f7f7f7f7f7f7full;
            dd += (uint32_t)__builtin_popcountll((((x & lo) + lo) | x) & ~lo);  // one flag per differing byte
        }
        return dd;
    }
#endif
    uint32_t d = 0;
    for (size_t r = 0; r < K; ++r) {
        const uint32_t ne = load_comp(a, comp_bytes, ia * K + r) != load_comp(b, comp_bytes, ib * K + r);
        d += r < g_primary ? ne << g_shift : ne;
    }
    return d;
}

// Legacy asymmetric_search_distance(CPQuery, CPCode), restated by hand in the reference at
// evaluation/debug_estimator.cpp:47-55: score = sum over r of (neg ? -val : val), distance = -score.
// DECLARED SUMMATION ORDER: the reference's scalar form adds r = 0..K-1 in sequence and its SIMD
// batch form adds in another order; the two agree only to 1e-5 (evaluation/qa_protocol.cpp:168-244).
// This oracle fixes one order, the balanced tree a 32-lane reduction produces: within each block
// of 32 rotations (missing terms are +0) term j is added to term j+16, then j+8, j+4, j+2, j+1;
// the block sums are added in sequence.  Within 1e-5 relative of the sequential sum.
inline float asym_dist(const float* table /*[K][P]*/, size_t K, size_t P, const void* codes,
                       size_t comp_bytes, size_t id) {
#if defined(CPHNSW_ORACLE_TUNED) && defined(__AVX512F__) && defined(__AVX512BW__) && defined(__AVX512VL__)
    // tuned build, 32 one-byte components: two 16-lane gathers and the same add tree (term j with j+16 is the sum
    // of the two vectors, then upper half onto lower half down to one lane), so the float is the plain build's
    if (K == 32 && comp_bytes == 1) {
        const __m256i c = _mm256_loadu_si256((const __m256i*)((const uint8_t*)codes + id * 32));
        const __m512i lo = _mm512_cvtepu8_epi32(_mm256_castsi256_si128(c));
        const __m512i hi = _mm512_cvtepu8_epi32(_mm256_extracti128_si256(c, 1));
        const __m512i lane = _mm512_set_epi32(15, 14, 13, 12, 11, 10, 9, 8, 7, 6, 5, 4, 3, 2, 1, 0);
        const __m512i p = _mm512_set1_epi32((int)P);
        const __m512i i0 = _mm512_add_epi32(_mm512_mullo_epi32(lane, p), _mm512_srli_epi32(lo, 1));
        const __m512i i1 = _mm512_add_epi32(_mm512_mullo_epi32(_mm512_add_epi32(lane, _mm512_set1_epi32(16)), p),
                                            _mm512_srli_epi32(hi, 1));
        __m512i v0 = _mm512_castps_si512(_mm512_i32gather_ps(i0, table, 4));
        __m512i v1 = _mm512_castps_si512(_mm512_i32gather_ps(i1, table, 4));
        v0 = _mm512_xor_si512(v0, _mm512_slli_epi32(lo, 31));  // odd component: negated
        v1 = _mm512_xor_si512(v1, _mm512_slli_epi32(hi, 31));
        const __m512 s16 = _mm512_add_ps(_mm512_castsi512_ps(v0), _mm512_castsi512_ps(v1));
        const __m256 s8 = _mm256_add_ps(_mm512_castps512_ps256(s16), _mm512_extractf32x8_ps(s16, 1));
        const __m128 s4 = _mm_add_ps(_mm256_castps256_ps128(s8), _mm256_extractf128_ps(s8, 1));
        const __m128 s2 = _mm_add_ps(s4, _mm_movehl_ps(s4, s4));
        const __m128 s1 = _mm_add_ss(s2, _mm_shuffle_ps(s2, s2, 1));
        return -(0.0f + _mm_cvtss_f32(s1));
    }
#endif
    float score = 0.0f;
    for (size_t c0 = 0; c0 < K; c0 += 32) {
        float t[32];
        for (size_t j = 0; j < 32; ++j) {
            size_t r = c0 + j;
            t[j] = 0.0f;
            if (r < K) {
                uint32_t c = load_comp(codes, comp_bytes, id * K + r);
                float val = table[r * P + (c >> 1)];
                t[j] = (c & 1) ? -val : val;
            }
        }
        for (size_t step = 16; step >= 1; step >>= 1)
            for (size_t j = 0; j < step; ++j) t[j] = t[j] + t[j + step];
        score = score + t[0];
    }
    return -score;
}

using Cand = std::pair<float, uint32_t>;  // total order (distance, id)

}  // namespace

extern "C" {

// include/cphnsw/encoder/rotation.hpp:134-144 (generate_signs) and :173-178 (rotation r is
// seeded base_seed + r): mt19937_64(seed), uniform_int_distribution<int>(0,1), layer-major draws.
// Output int8 [K][3][P].
int orc_sign_tables(uint64_t dim, uint64_t K, uint64_t seed, int8_t* out) {
    size_t P = next_pow2(dim);
    for (size_t r = 0; r < K; ++r) {
        std::mt19937_64 rng(seed + r);
        std::uniform_int_distribution<int> coin(0, 1);
        for (int layer = 0; layer < 3; ++layer)
            for (size_t i = 0; i < P; ++i) out[(r * 3 + layer) * P + i] = coin(rng) ? 1 : -1;
    }
    return 0;
}

int orc_fht(float* v, uint64_t n, int convention) {
    fht_convention(v, n, convention);
    return 0;
}

// Legacy CPEncoder<ComponentT,K>::encode (absent); loop structure from
// include/cphnsw/encoder/cp_encoder.hpp:161-184, byte format from types.hpp:88-90 and
// src/cuda/gpu_encoder.cu:214-218.  Sign test `buffer[idx] < 0` (cp_encoder.hpp:174).
// Optional outputs: rotated [n][K][P], magnitudes [n][K] (CPQuery, types.hpp:324-337).
int orc_encode(const float* x, uint64_t n, uint64_t dim, uint64_t K, uint64_t comp_bytes,
               const int8_t* signs, int convention, void* codes, float* rotated, float* magnitudes) {
    size_t P = next_pow2(dim);
#pragma omp parallel
    {
        std::vector<float> buf(P);
#pragma omp for schedule(static)
        for (int64_t i = 0; i < (int64_t)n; ++i)
            for (size_t r = 0; r < K; ++r) {
                rotate(x + (size_t)i * dim, dim, P, signs + r * 3 * P, convention, buf.data());
                size_t idx;
                float mag;
                argmax_abs(buf.data(), P, idx, mag);
                store_comp(codes, comp_bytes, (size_t)i * K + r, component(idx, buf[idx] < 0));
                if (rotated) std::memcpy(rotated + ((size_t)i * K + r) * P, buf.data(), P * sizeof(float));
                if (magnitudes) magnitudes[(size_t)i * K + r] = mag;
            }
    }
    return 0;
}

int orc_set_residual_weighting(uint64_t primary_components, uint32_t shift) {
    g_primary = primary_components;
    g_shift = shift;
    return 0;
}

// All-pairs code distance, out[na][nb] uint16 (HammingDist, types.hpp:35).
int orc_code_distance(const void* a, uint64_t na, const void* b, uint64_t nb, uint64_t K,
                      uint64_t comp_bytes, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)na; ++i)
        for (size_t j = 0; j < nb; ++j)
            out[(size_t)i * nb + j] = (uint16_t)code_dist(a, i, b, j, K, comp_bytes);
    return 0;
}

// Brute-force code-distance kNN rows [row_begin,row_end) against all n codes: self excluded,
// k smallest under (distance, id); rows with fewer than k candidates are padded with
// 0xFFFFFFFF / 0xFFFF (padding convention of src/cuda/gpu_knn_graph.cu:154-181).
int orc_knn_graph(const void* codes, uint64_t n, uint64_t K, uint64_t comp_bytes, uint64_t k,
                  uint64_t row_begin, uint64_t row_end, uint32_t* nbrs, uint16_t* dists) {
#pragma omp parallel
    {
        std::vector<std::pair<uint32_t, uint32_t>> best;  // (dist, id) ascending, size <= k
#pragma omp for schedule(dynamic, 16)
        for (int64_t i = (int64_t)row_begin; i < (int64_t)row_end; ++i) {
            best.clear();
            for (size_t j = 0; j < n; ++j) {
                if ((size_t)i == j) continue;
                uint32_t d = code_dist(codes, i, codes, j, K, comp_bytes);
                // j ascends, so a later id never displaces an equal distance
                if (best.size() == k && d >= best.back().first) continue;
                auto it = std::upper_bound(best.begin(), best.end(), std::make_pair(d, (uint32_t)j));
                best.insert(it, {d, (uint32_t)j});
                if (best.size() > k) best.pop_back();
            }
            size_t o = ((size_t)i - row_begin) * k;
            for (size_t t = 0; t < k; ++t) {
                nbrs[o + t] = t < best.size() ? best[t].second : kInvalid;
                if (dists) dists[o + t] = t < best.size() ? (uint16_t)best[t].first : (uint16_t)0xFFFF;
            }
        }
    }
    return 0;
}

// SELECT-NEIGHBORS-HEURISTIC with keepPrunedConnections
// (resources/hnsw-paper/consolidated.tex:93-115; flag default types.hpp:390-391).
// Candidates of row i are cand[i][0..k) in the order given (ascending (distance,id) from the
// kNN build); "closer" is strict < on the integer code distance.  Output adj[rows][M].
int orc_select_neighbors(const void* codes, uint64_t n, uint64_t K, uint64_t comp_bytes,
                         const uint32_t* cand, uint64_t k, uint64_t M, int keep_pruned,
                         uint64_t row_begin, uint64_t row_end, uint32_t* adj) {
    (void)n;
#pragma omp parallel for schedule(static)
    for (int64_t i = (int64_t)row_begin; i < (int64_t)row_end; ++i) {
        const uint32_t* c = cand + ((size_t)i - row_begin) * k;
        uint32_t* out = adj + ((size_t)i - row_begin) * M;
        std::vector<uint32_t> R, Wd;
        for (size_t t = 0; t < k && R.size() < M; ++t) {
            uint32_t e = c[t];
            if (e == kInvalid) continue;
            uint32_t d_eq = code_dist(codes, e, codes, i, K, comp_bytes);
            bool keep = true;
            for (uint32_t r : R)
                if (!(d_eq < code_dist(codes, e, codes, r, K, comp_bytes))) {
                    keep = false;
                    break;
                }
            (keep ? R : Wd).push_back(e);
        }
        if (keep_pruned)
            for (size_t t = 0; t < Wd.size() && R.size() < M; ++t) R.push_back(Wd[t]);
        for (size_t t = 0; t < M; ++t) out[t] = t < R.size() ? R[t] : kInvalid;
    }
    return 0;
}

// Beam search over a flat adjacency; control flow of
// include/cphnsw/search/search_engine.hpp:86-193 with two declared differences:
//  * candidates are compared under the total order (distance, id), so the result does not depend
//    on heap insertion order (the reference compares `distance` only, types.hpp:351-357);
//  * the best k of W are returned ascending (the reference pops the k worst, :184-190; the
//    legacy behaviour asserted by evaluation/qa_protocol.cpp:137-165 is ascending best-k).
// Metric: legacy asymmetric distance against the query's K rotated vectors (table).
// Entry: every id of entry_ids is scored (the "entry scan"); the n_seed best under (distance, id)
// seed the walk - the legacy index's k_entry entry points (types.hpp:396-397), chosen by score
// instead of at random so that a query lands in its own cluster.  n_seed >= n_entry offers them all.
// W capacity is ef.  out_ids/out_dist are [nq][k] padded with 0xFFFFFFFF / +inf; stats[nq][2] =
// expansions, distance evaluations (scan + walk; optional).
}  // extern "C"

namespace {
// dist_of(q, id) is the metric: the asymmetric CP score for search / search_and_rerank, the
// symmetric code distance to a probe code for search_multiprobe.
template <class DistFn>
int walk_all(uint64_t nq, uint64_t n, const uint32_t* adj, uint64_t M, const uint32_t* entry_ids, uint64_t n_entry,
             uint64_t n_seed, uint64_t ef, uint64_t k, uint32_t* out_ids, float* out_dist, uint32_t* stats,
             DistFn dist_of) {
#ifdef CPHNSW_ORACLE_TUNED
    // Tuned build: the same walk with W as one sorted array (binary search + shift on admission, an
    // "expanded" flag per member, a cursor on the first unexpanded member) and an epoch-stamped visited
    // array, instead of two std::set.  Same total order, so the same results; the plain build is the checker.
#pragma omp parallel
    {
        std::vector<uint32_t> stamp(n, 0u);
        uint32_t epoch = 0;
        struct Member {
            float d;
            uint32_t id;
            bool expanded;
        };
        std::vector<Member> W;
        W.reserve(ef + 1);
#pragma omp for schedule(dynamic, 4)
        for (int64_t q = 0; q < (int64_t)nq; ++q) {
            if (++epoch == 0) {
                std::fill(stamp.begin(), stamp.end(), 0u);
                epoch = 1;
            }
            W.clear();
            size_t cur = 0;  // no unexpanded member before this position
            uint32_t expansions = 0, evals = 0;
            auto offer = [&](uint32_t id) {
                if (id == kInvalid || id >= n || stamp[id] == epoch) return;
                stamp[id] = epoch;
                const float d = dist_of((size_t)q, id);
                ++evals;
                if (W.size() == ef && !(Cand{d, id} < Cand{W.back().d, W.back().id})) return;
                size_t lo = 0, hi = W.size();
                while (lo < hi) {
                    const size_t mid = (lo + hi) / 2;
                    if (Cand{W[mid].d, W[mid].id} < Cand{d, id}) lo = mid + 1;
                    else hi = mid;
                }
                if (W.size() == ef) W.pop_back();
                W.insert(W.begin() + lo, Member{d, id, false});
                if (lo < cur) cur = lo;
            };
            if (n_seed >= n_entry) {
                for (size_t e = 0; e < n_entry; ++e) offer(entry_ids[e]);
            } else {
                std::vector<Cand> scan;
                scan.reserve(n_entry);
                for (size_t e = 0; e < n_entry; ++e) {
                    const uint32_t id = entry_ids[e];
                    if (id == kInvalid || id >= n) continue;
                    scan.push_back({dist_of((size_t)q, id), id});
                    ++evals;
                }
                // the n_seed best without sorting everything; a full sort only if repeated ids ate the margin
                size_t keep = std::min<size_t>(scan.size(), 2 * n_seed + 8);
                std::partial_sort(scan.begin(), scan.begin() + keep, scan.end());
                std::vector<Cand> head(scan.begin(), scan.begin() + keep);
                head.erase(std::unique(head.begin(), head.end()), head.end());
                if (head.size() < n_seed && keep < scan.size()) {
                    std::sort(scan.begin(), scan.end());
                    scan.erase(std::unique(scan.begin(), scan.end()), scan.end());
                } else {
                    scan.swap(head);
                }
                for (size_t e = 0; e < scan.size() && e < n_seed; ++e) offer(scan[e].second);
            }
            for (;;) {
                while (cur < W.size() && W[cur].expanded) ++cur;
                if (cur == W.size()) break;
                W[cur].expanded = true;
                ++expansions;
                const uint32_t* row = adj + (size_t)W[cur].id * M;
                for (size_t t = 0; t < M; ++t) offer(row[t]);
            }
            const size_t o = (size_t)q * k;
            size_t t = 0;
            for (; t < k && t < W.size(); ++t) {
                out_ids[o + t] = W[t].id;
                out_dist[o + t] = W[t].d;
            }
            for (; t < k; ++t) {
                out_ids[o + t] = kInvalid;
                out_dist[o + t] = INFINITY;
            }
            if (stats) {
                stats[2 * q] = expansions;
                stats[2 * q + 1] = evals;
            }
        }
    }
#else
#pragma omp parallel
    {
        std::vector<uint8_t> visited(n);
        std::vector<uint32_t> touched;
#pragma omp for schedule(dynamic, 4)
        for (int64_t q = 0; q < (int64_t)nq; ++q) {
            std::set<Cand> W;  // at most ef best seen so far
            std::set<Cand> C;  // members of W not yet expanded
            uint32_t expansions = 0, evals = 0;
            auto offer = [&](uint32_t id) {
                if (id == kInvalid || id >= n || visited[id]) return;  // search_engine.hpp:154-160
                visited[id] = 1;
                touched.push_back(id);
                Cand c{dist_of((size_t)q, id), id};
                ++evals;
                if (W.size() < ef) {  // search_engine.hpp:166-176
                    W.insert(c);
                    C.insert(c);
                } else if (c < *W.rbegin()) {
                    Cand worst = *W.rbegin();
                    W.erase(worst);
                    C.erase(worst);
                    W.insert(c);
                    C.insert(c);
                }
            };
            if (n_seed >= n_entry) {
                for (size_t e = 0; e < n_entry; ++e) offer(entry_ids[e]);  // :105-115
            } else {
                std::vector<Cand> scan;
                for (size_t e = 0; e < n_entry; ++e) {
                    uint32_t id = entry_ids[e];
                    if (id == kInvalid || id >= n) continue;
                    scan.push_back({dist_of((size_t)q, id), id});
                    ++evals;
                }
                std::sort(scan.begin(), scan.end());
                scan.erase(std::unique(scan.begin(), scan.end()), scan.end());
                for (size_t e = 0; e < scan.size() && e < n_seed; ++e) offer(scan[e].second);
            }
            while (!C.empty()) {  // :118-178; C only holds members of W, so the `c > worst` break
                Cand c = *C.begin();  // of :130-132 is the emptiness of C
                C.erase(C.begin());
                ++expansions;
                const uint32_t* row = adj + (size_t)c.second * M;
                for (size_t t = 0; t < M; ++t) offer(row[t]);
            }
            size_t o = (size_t)q * k, t = 0;
            for (auto it = W.begin(); it != W.end() && t < k; ++it, ++t) {
                out_ids[o + t] = it->second;
                out_dist[o + t] = it->first;
            }
            for (; t < k; ++t) {
                out_ids[o + t] = kInvalid;
                out_dist[o + t] = INFINITY;
            }
            if (stats) {
                stats[2 * q] = expansions;
                stats[2 * q + 1] = evals;
            }
            for (uint32_t id : touched) visited[id] = 0;
            touched.clear();
        }
    }
#endif
    return 0;
}
}  // namespace

extern "C" {

int orc_search(const float* tables /*[nq][K][P]*/, uint64_t nq, uint64_t K, uint64_t P,
               const void* codes, uint64_t comp_bytes, uint64_t n, const uint32_t* adj, uint64_t M,
               const uint32_t* entry_ids, uint64_t n_entry, uint64_t n_seed, uint64_t ef, uint64_t k,
               uint32_t* out_ids, float* out_dist, uint32_t* stats) {
    return walk_all(nq, n, adj, M, entry_ids, n_entry, n_seed, ef, k, out_ids, out_dist, stats,
                    [&](size_t q, uint32_t id) { return asym_dist(tables + q * K * P, K, P, codes, comp_bytes, id); });
}

// The same walk under the symmetric metric: distance = number of components in which the node's
// code differs from the query's code qcodes[q] (legacy hamming_distance), as a float.
int orc_search_codes(const void* qcodes /*[nq][K]*/, uint64_t nq, uint64_t K, const void* codes,
                     uint64_t comp_bytes, uint64_t n, const uint32_t* adj, uint64_t M, const uint32_t* entry_ids,
                     uint64_t n_entry, uint64_t n_seed, uint64_t ef, uint64_t k, uint32_t* out_ids, float* out_dist,
                     uint32_t* stats) {
    return walk_all(nq, n, adj, M, entry_ids, n_entry, n_seed, ef, k, out_ids, out_dist, stats,
                    [&](size_t q, uint32_t id) { return (float)code_dist(qcodes, q, codes, id, K, comp_bytes); });
}

// Multiprobe sequence for the cross-polytope hash (resources/cross-polytope-lsh/consolidated.tex:391-425;
// data kept for it in CPQuery, types.hpp:332-336).  Per rotation the coordinates are ranked by
// (|x| descending, index ascending); replacing the winner by the coordinate of rank v costs
// (|x|_(0) - |x|_(v))^2 (the paper's single-coordinate approximation); a probe is a choice of one
// rank per rotation, scored by the sum of its costs over rotations in ascending rotation order
// (fp32).  Probes are emitted in ascending (score, creation number) order, the primary code first:
// after emitting a probe whose last modified rotation is j, its successors are "raise the rank of
// rotation j by one" and "set rotation j' to rank 1" for every j' > j (each probe has exactly one
// such derivation).  rotated is [nq][K][P]; probe codes out [nq][T][K].
int orc_probe_codes(const float* rotated, uint64_t nq, uint64_t K, uint64_t P, uint64_t comp_bytes, uint64_t T,
                    void* out) {
    const size_t V = std::min<size_t>(P, T + 1);  // ranks that T probes can reach
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < (int64_t)nq; ++q) {
        std::vector<uint32_t> idx(K * V);
        std::vector<float> cost(K * V);
        for (size_t r = 0; r < K; ++r) {
            const float* x = rotated + ((size_t)q * K + r) * P;
            std::vector<std::pair<float, uint32_t>> key(P);
            for (size_t i = 0; i < P; ++i) key[i] = {-std::fabs(x[i]), (uint32_t)i};
            std::partial_sort(key.begin(), key.begin() + V, key.end());
            const float top = -key[0].first;
            for (size_t v = 0; v < V; ++v) {
                idx[r * V + v] = key[v].second;
                float d = top - (-key[v].first);
                cost[r * V + v] = d * d;
            }
        }
        struct Item { float score; uint32_t seq, parent, rot, rank; bool used; };
        std::vector<Item> pool;
        std::vector<std::vector<uint8_t>> ranks;  // emitted probes
        std::vector<uint32_t> last;                // last modified rotation of each emitted probe
        auto score_of = [&](const std::vector<uint8_t>& rk) {
            float s = 0.0f;
            for (size_t r = 0; r < K; ++r)
                if (rk[r]) s = s + cost[r * V + rk[r]];
            return s;
        };
        auto push_children = [&](uint32_t parent) {
            const std::vector<uint8_t>& rk = ranks[parent];
            const bool primary = parent == 0;
            uint32_t j = primary ? 0 : last[parent];
            if (!primary && (size_t)rk[j] + 1 < V) {
                std::vector<uint8_t> c = rk;
                c[j] = rk[j] + 1;
                pool.push_back({score_of(c), (uint32_t)pool.size(), parent, j, (uint32_t)c[j], false});
            }
            for (uint32_t j2 = primary ? 0 : j + 1; j2 < K; ++j2) {
                if (V < 2) break;
                std::vector<uint8_t> c = rk;
                c[j2] = 1;
                pool.push_back({score_of(c), (uint32_t)pool.size(), parent, j2, 1u, false});
            }
        };
        ranks.push_back(std::vector<uint8_t>(K, 0));
        last.push_back(0);
        push_children(0);
        while (ranks.size() < T) {
            int best = -1;
            for (size_t i = 0; i < pool.size(); ++i)
                if (!pool[i].used && (best < 0 || pool[i].score < pool[best].score)) best = (int)i;  // lowest seq wins ties
            if (best < 0) break;  // fewer than T distinct probes exist
            pool[best].used = true;
            std::vector<uint8_t> rk = ranks[pool[best].parent];
            rk[pool[best].rot] = (uint8_t)pool[best].rank;
            ranks.push_back(rk);
            last.push_back(pool[best].rot);
            push_children((uint32_t)ranks.size() - 1);
        }
        for (size_t t = 0; t < T; ++t) {
            const std::vector<uint8_t>& rk = ranks[std::min(t, ranks.size() - 1)];  // repeat the last probe if short
            for (size_t r = 0; r < K; ++r) {
                uint32_t i = idx[r * V + rk[r]];
                float val = rotated[((size_t)q * K + r) * P + i];
                store_comp(out, comp_bytes, ((size_t)q * T + t) * K + r, component(i, val < 0));
            }
        }
    }
    return 0;
}

// Merge of the per-probe result lists of search_multiprobe: per query, the union of T lists of k
// (id, distance), each id kept once with its smallest distance, ascending by (distance, id), best k.
int orc_merge_probes(const uint32_t* ids /*[nq][T][k]*/, const float* dist, uint64_t nq, uint64_t T, uint64_t k,
                     uint32_t* out_ids, float* out_dist) {
    for (size_t q = 0; q < nq; ++q) {
        std::vector<std::pair<uint32_t, float>> all;
        for (size_t i = 0; i < T * k; ++i)
            if (ids[q * T * k + i] != kInvalid) all.push_back({ids[q * T * k + i], dist[q * T * k + i]});
        std::sort(all.begin(), all.end());
        std::vector<Cand> best;
        for (size_t i = 0; i < all.size(); ++i)
            if (i == 0 || all[i].first != all[i - 1].first) best.push_back({all[i].second, all[i].first});
        std::sort(best.begin(), best.end());
        for (size_t t = 0; t < k; ++t) {
            out_ids[q * k + t] = t < best.size() ? best[t].second : kInvalid;
            out_dist[q * k + t] = t < best.size() ? best[t].first : INFINITY;
        }
    }
    return 0;
}

// Exact rerank of candidate ids: distance = -<q, x_id> accumulated in d order in fp32
// (evaluation/eval_sift.cpp:539-563), sort ascending by (distance, id), keep k.
// cand is [nq][n_cand] (0xFFFFFFFF entries skipped).
int orc_rerank(const float* queries, uint64_t nq, uint64_t dim, const float* base,
               const uint32_t* cand, uint64_t n_cand, uint64_t k, uint32_t* out_ids, float* out_dist) {
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t q = 0; q < (int64_t)nq; ++q) {
        std::vector<Cand> r;
        for (size_t t = 0; t < n_cand; ++t) {
            uint32_t id = cand[(size_t)q * n_cand + t];
            if (id == kInvalid) continue;
            float dot = 0.0f;
            for (size_t d = 0; d < dim; ++d) dot += queries[(size_t)q * dim + d] * base[(size_t)id * dim + d];
            r.push_back({-dot, id});
        }
        std::sort(r.begin(), r.end());
        for (size_t t = 0; t < k; ++t) {
            out_ids[(size_t)q * k + t] = t < r.size() ? r[t].second : kInvalid;
            out_dist[(size_t)q * k + t] = t < r.size() ? r[t].first : INFINITY;
        }
    }
    return 0;
}

// Exact cosine ground truth for unit vectors (evaluation/datasets/dataset_loader.hpp:187-212;
// GPUBruteForce::search, src/cuda/gpu_encoder.cu:554-603): top-k by (-dot, id); out_dist may be null.
int orc_ground_truth(const float* queries, uint64_t nq, const float* base, uint64_t n, uint64_t dim,
                     uint64_t k, uint32_t* out_ids, float* out_dist) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t q = 0; q < (int64_t)nq; ++q) {
        std::vector<Cand> best;
        for (size_t i = 0; i < n; ++i) {
            float dot = 0.0f;
            for (size_t d = 0; d < dim; ++d) dot += queries[(size_t)q * dim + d] * base[i * dim + d];
            Cand c{-dot, (uint32_t)i};
            if (best.size() == k && !(c < best.back())) continue;
            best.insert(std::upper_bound(best.begin(), best.end(), c), c);
            if (best.size() > k) best.pop_back();
        }
        for (size_t t = 0; t < k; ++t) {
            out_ids[(size_t)q * k + t] = t < best.size() ? best[t].second : kInvalid;
            if (out_dist) out_dist[(size_t)q * k + t] = t < best.size() ? best[t].first : INFINITY;
        }
    }
    return 0;
}

// Diagnostics of the legacy index.  Their sources are absent from the reference tree; the
// behaviour is restated from the call sites.
//
// brute_force_search (evaluation/eval_sift.cpp:283,329; test_k_variants.cpp:79): the k nodes with
// the smallest asymmetric CP score among all n, ascending by (score, id).
int orc_brute_force(const float* tables /*[nq][K][P]*/, uint64_t nq, uint64_t K, uint64_t P, const void* codes,
                    uint64_t comp_bytes, uint64_t n, uint64_t k, uint32_t* out_ids, float* out_dist) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t q = 0; q < (int64_t)nq; ++q) {
        const float* table = tables + (size_t)q * K * P;
        std::vector<Cand> best;
        for (size_t i = 0; i < n; ++i) {
            Cand c{asym_dist(table, K, P, codes, comp_bytes, i), (uint32_t)i};
            if (best.size() == k && !(c < best.back())) continue;
            best.insert(std::upper_bound(best.begin(), best.end(), c), c);
            if (best.size() > k) best.pop_back();
        }
        for (size_t t = 0; t < k; ++t) {
            out_ids[(size_t)q * k + t] = t < best.size() ? best[t].second : kInvalid;
            out_dist[(size_t)q * k + t] = t < best.size() ? best[t].first : INFINITY;
        }
    }
    return 0;
}

// calibrate(num_samples, seed) (evaluation/eval_main.cpp:128-135, qa_protocol.cpp:263-270): pairs
// (u, v) of stored nodes drawn with std::mt19937_64(seed) (u = next() % n, then v = next() % n);
// x = asymmetric CP score of v's code for u as the query, y = -<x_u, x_v> accumulated in d order
// in fp32.  Outputs the pairs and the samples; the least-squares fit is orc_linear_fit.
int orc_calibration_samples(const float* tables /*[num_samples][K][P] of the u vectors, in sample order*/,
                            uint64_t K, uint64_t P, const void* codes, uint64_t comp_bytes, const float* base,
                            uint64_t n, uint64_t dim, uint64_t num_samples, const uint32_t* u, const uint32_t* v,
                            float* x, float* y) {
#pragma omp parallel for schedule(static)
    for (int64_t s = 0; s < (int64_t)num_samples; ++s) {
        x[s] = asym_dist(tables + (size_t)s * K * P, K, P, codes, comp_bytes, v[s]);
        float dot = 0.0f;
        for (size_t d = 0; d < dim; ++d) dot += base[(size_t)u[s] * dim + d] * base[(size_t)v[s] * dim + d];
        y[s] = -dot;
    }
    (void)n;
    return 0;
}

int orc_calibration_pairs(uint64_t n, uint64_t num_samples, uint64_t seed, uint32_t* u, uint32_t* v) {
    std::mt19937_64 rng(seed);
    for (uint64_t s = 0; s < num_samples; ++s) {
        u[s] = (uint32_t)(rng() % n);
        v[s] = (uint32_t)(rng() % n);
    }
    return 0;
}

// y ~ alpha * x + beta by least squares in double; r_squared = squared correlation (0 when x or y
// is constant).  out = {alpha, beta, r_squared}.
int orc_linear_fit(const float* x, const float* y, uint64_t m, double* out) {
    double sx = 0, sy = 0;
    for (uint64_t i = 0; i < m; ++i) sx += x[i], sy += y[i];
    const double mx = m ? sx / m : 0, my = m ? sy / m : 0;
    double sxx = 0, sxy = 0, syy = 0;
    for (uint64_t i = 0; i < m; ++i) {
        const double dx = x[i] - mx, dy = y[i] - my;
        sxx += dx * dx, sxy += dx * dy, syy += dy * dy;
    }
    const double alpha = sxx > 0 ? sxy / sxx : 0.0;
    out[0] = alpha;
    out[1] = my - alpha * mx;
    out[2] = (sxx > 0 && syy > 0) ? (sxy * sxy) / (sxx * syy) : 0.0;
    return 0;
}

// verify_connectivity() (evaluation/eval_main.cpp:52, eval_sift.cpp:266): number of nodes reachable
// from the entry nodes along the directed adjacency (the entry nodes included).
uint64_t orc_connectivity(const uint32_t* adj, uint64_t n, uint64_t M, const uint32_t* entry_ids, uint64_t n_entry) {
    std::vector<uint8_t> seen(n, 0);
    std::vector<uint32_t> stack;
    uint64_t count = 0;
    for (uint64_t e = 0; e < n_entry; ++e)
        if (entry_ids[e] < n && !seen[entry_ids[e]]) seen[entry_ids[e]] = 1, stack.push_back(entry_ids[e]), ++count;
    while (!stack.empty()) {
        const uint32_t v = stack.back();
        stack.pop_back();
        for (uint64_t j = 0; j < M; ++j) {
            const uint32_t w = adj[(size_t)v * M + j];
            if (w < n && !seen[w]) seen[w] = 1, stack.push_back(w), ++count;
        }
    }
    return count;
}

// Rank-based pruning of kNN lists (CAGRA graph optimisation; the legacy build_with_gpu_knn(..., prune,
// alpha), evaluation/test_gpu_build.cpp:168-174, parameter include/cphnsw/core/types.hpp:399-400; rule
// resources/arXiv-2308.15136v2/consolidated.tex:298-340).  cand[n][k] in ascending (distance, id) order.
//   reorder: detours of edge X -> Y = #{Z in L_X : Y in L_Z and alpha * max(rank_X(Z), rank_Z(Y)) < rank_X(Y)},
//            ranks 1-based, the product in fp32; keep the M first by (detours, rank).
//   reverse: P receives the X that kept P, ordered by (position of P in X's kept list, X), at most M.
//   merge:   interleave kept and reverse list, kept first, each id once, until M; an exhausted list
//            passes its turns to the other.
int orc_rank_prune(const uint32_t* cand, uint64_t n, uint64_t k, uint64_t M, float alpha, uint32_t* adj) {
    std::vector<uint32_t> kept(n * M, kInvalid);
#pragma omp parallel for schedule(static)
    for (int64_t x = 0; x < (int64_t)n; ++x) {
        const uint32_t* lx = cand + (size_t)x * k;
        std::vector<std::pair<uint32_t, uint32_t>> order;  // (detours, position)
        for (size_t j = 0; j < k; ++j) {
            const uint32_t y = lx[j];
            if (y >= n) continue;
            uint32_t detours = 0;
            for (size_t i = 0; i < k; ++i) {
                const uint32_t z = lx[i];
                if (z >= n) continue;
                const uint32_t* lz = cand + (size_t)z * k;
                for (size_t p = 0; p < k; ++p)
                    if (lz[p] == y) {
                        const float thr = alpha * (float)(std::max(i, p) + 1);
                        if (thr < (float)(j + 1)) ++detours;
                    }
            }
            order.push_back({detours, (uint32_t)j});
        }
        std::sort(order.begin(), order.end());
        for (size_t t = 0; t < order.size() && t < M; ++t) kept[(size_t)x * M + t] = lx[order[t].second];
    }
    std::vector<std::vector<std::pair<uint32_t, uint32_t>>> rev(n);  // (position in the chooser's list, chooser)
    for (size_t x = 0; x < n; ++x)
        for (size_t r = 0; r < M; ++r) {
            const uint32_t p = kept[x * M + r];
            if (p < n) rev[p].push_back({(uint32_t)r, (uint32_t)x});
        }
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < (int64_t)n; ++p) {
        std::sort(rev[p].begin(), rev[p].end());
        if (rev[p].size() > M) rev[p].resize(M);
        std::vector<uint32_t> a, b, out;
        for (size_t r = 0; r < M; ++r)
            if (kept[(size_t)p * M + r] < n) a.push_back(kept[(size_t)p * M + r]);
        for (auto& e : rev[p]) b.push_back(e.second);
        size_t ia = 0, ib = 0;
        int turn = 0;
        auto taken = [&](uint32_t id) { return std::find(out.begin(), out.end(), id) != out.end(); };
        while (out.size() < M) {
            while (ia < a.size() && taken(a[ia])) ++ia;
            while (ib < b.size() && taken(b[ib])) ++ib;
            if (ia >= a.size() && ib >= b.size()) break;
            const bool from_a = ib >= b.size() || (ia < a.size() && turn == 0);
            out.push_back(from_a ? a[ia++] : b[ib++]);
            turn ^= 1;
        }
        for (size_t t = 0; t < M; ++t) adj[(size_t)p * M + t] = t < out.size() ? out[t] : kInvalid;
    }
    return 0;
}

// Links chosen on the fp32 vectors: the legacy "hybrid" construction ("Hybrid (True Cosine edges) - the production
// path", evaluation/eval_master.cpp:251-272; evaluation/test_tiered.cpp:4-7; source absent).
// distance(a, b) = -<a, b>, products and sums separate, summed in d order (the loop of evaluation/eval_sift.cpp:546-551).
static inline float neg_dot(const float* a, const float* b, size_t dim) {
    float acc = 0.0f;
    for (size_t d = 0; d < dim; ++d) acc = acc + a[d] * b[d];
    return -acc;
}

// Candidates of row i: the exact top-(k+1) of ALL vectors by (distance to x_i, id) with i itself removed, cut to k
// (i is in its own list unless more than k exact duplicates with lower ids precede it).
int orc_exact_candidates(const float* base, uint64_t n, uint64_t dim, uint64_t k, uint64_t row_begin, uint64_t row_end,
                         uint32_t* cand) {
#pragma omp parallel for schedule(dynamic, 8)
    for (int64_t i = (int64_t)row_begin; i < (int64_t)row_end; ++i) {
        std::vector<Cand> all(n);
        for (size_t j = 0; j < n; ++j) all[j] = {neg_dot(base + (size_t)i * dim, base + j * dim, dim), (uint32_t)j};
        const size_t keep = std::min<size_t>(n, k + 1);
        std::partial_sort(all.begin(), all.begin() + keep, all.end());
        uint32_t* out = cand + ((size_t)i - row_begin) * k;
        size_t o = 0;
        for (size_t t = 0; t < keep && o < k; ++t)
            if (all[t].second != (uint32_t)i) out[o++] = all[t].second;
        for (; o < k; ++o) out[o] = kInvalid;
    }
    return 0;
}

// SELECT-NEIGHBORS-HEURISTIC with keepPrunedConnections on those exact distances
// (resources/hnsw-paper/consolidated.tex:93-115): candidate e is kept iff d(e, q) < d(e, r) for every r kept so far.
int orc_select_neighbors_exact(const float* base, uint64_t n, uint64_t dim, const uint32_t* cand, uint64_t k, uint64_t M,
                               int keep_pruned, uint64_t row_begin, uint64_t row_end, uint32_t* adj) {
#pragma omp parallel for schedule(static)
    for (int64_t i = (int64_t)row_begin; i < (int64_t)row_end; ++i) {
        const uint32_t* c = cand + ((size_t)i - row_begin) * k;
        uint32_t* out = adj + ((size_t)i - row_begin) * M;
        std::vector<uint32_t> R, Wd;
        for (size_t t = 0; t < k && R.size() < M; ++t) {
            const uint32_t e = c[t];
            if (e >= n) continue;
            const float d_eq = neg_dot(base + (size_t)e * dim, base + (size_t)i * dim, dim);
            bool keep = true;
            for (uint32_t r : R)
                if (!(d_eq < neg_dot(base + (size_t)e * dim, base + (size_t)r * dim, dim))) {
                    keep = false;
                    break;
                }
            (keep ? R : Wd).push_back(e);
        }
        if (keep_pruned)
            for (size_t t = 0; t < Wd.size() && R.size() < M; ++t) R.push_back(Wd[t]);
        for (size_t t = 0; t < M; ++t) out[t] = t < R.size() ? R[t] : kInvalid;
    }
    return 0;
}

// Thread count of every parallel region from now on (launchers such as torchrun export OMP_NUM_THREADS=1).
int orc_set_threads(int threads) {
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
    return omp_get_max_threads();
#else
    (void)threads;
    return 1;
#endif
}

// 1 when this library is the tuned build (the benchmark's CPU baseline), 0 for the plain checker.
int orc_is_tuned() {
#ifdef CPHNSW_ORACLE_TUNED
    return 1;
#else
    return 0;
#endif
}

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
