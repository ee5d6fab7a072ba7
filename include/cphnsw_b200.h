/*
 * cphnsw_b200 — C ABI of the B200 (sm_100a) implementation of the CP-HNSW data-parallel hot path:
 * cross-polytope encode, CP-code distance, brute-force code-distance kNN graph, select_neighbors
 * pruning, batched beam search and exact rerank.
 *
 * Conventions
 *   - every function returns 0 on success or a negative CPHNSW_B200_E_* code; nothing exits,
 *     aborts or throws.  cphnsw_b200_last_error() gives the message of the last failure on
 *     the calling thread.
 *   - plain entry points take caller-owned HOST pointers (row-major, not retained) and do their
 *     own host<->device copies, like the reference's GPU classes do
 *     (include/cphnsw/cuda/gpu_encoder.cuh:24-93, include/cphnsw/cuda/gpu_knn_graph.cuh:28-101).
 *   - "_dev" entry points take DEVICE pointers on the index's device and a cudaStream_t passed
 *     as void*; they are asynchronous on that stream and allocate no output.
 *   - a handle is bound to one CUDA device and is thread-safe.  The search entry points (search_batch,
 *     search_and_rerank_batch, search_multiprobe_batch, brute_force_search_batch, search_calibrated_batch,
 *     search_codes_batch, search_dev) run concurrently from any number of host threads, as the reference's
 *     callers do from OpenMP loops (evaluation/eval_sift.cpp:279-283,380-387,423-430): each call works in a
 *     search context of its own (stream, staging buffers, visited slots) taken from a pool in the handle.
 *     Calls of up to 32 queries get one thread block per query and up to 64 of them run side by side; larger
 *     batches fill the GPU and take turns.  Every other entry point (add*, install, set_param, the stage
 *     calls, save) excludes all others while it runs, like the mutex of the reference's add
 *     (include/cphnsw/graph/flat_graph.hpp:80-98).
 *   - code layout is row-major ComponentT[n][K], component = (argmax_index << 1) | negative
 *     (include/cphnsw/core/types.hpp:68-106).  Node ids are uint32, 0xFFFFFFFF is "no node"
 *     (types.hpp:28-30).
 *
 * The library has no CPU fallback: every entry point fails with CPHNSW_B200_E_CUDA when no
 * sm_100 device is usable.
 */
#ifndef CPHNSW_B200_H
#define CPHNSW_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CPHNSW_B200_OK 0
#define CPHNSW_B200_E_INVALID (-1)   /* bad argument (maps to std::invalid_argument, types.hpp:409-457) */
#define CPHNSW_B200_E_CUDA (-2)      /* CUDA runtime error or no usable device */
#define CPHNSW_B200_E_STATE (-3)     /* call not valid in the index's current state (e.g. search before build) */
#define CPHNSW_B200_E_UNSUPPORTED (-4)
#define CPHNSW_B200_E_DEVICE_WAIT (-5) /* a bounded device-side wait ran out; the context stays usable */

/* FHT sign convention of the reference build being matched
 * (include/cphnsw/encoder/transform/fht.hpp:56-69 scalar, :81-127 AVX2, :141-196 AVX-512). */
#define CPHNSW_B200_FHT_SCALAR 0
#define CPHNSW_B200_FHT_AVX2 1
#define CPHNSW_B200_FHT_AVX512 2

#define CPHNSW_B200_INVALID_NODE 0xFFFFFFFFu

typedef struct cphnsw_b200_index cphnsw_b200_index;

const char* cphnsw_b200_last_error(void);

/* Number of usable sm_100 devices (0 when none / no driver).  Never fails. */
int cphnsw_b200_device_count(void);

/* ---- lifetime -------------------------------------------------------------------------------
 * Replaces the constructors CPHNSWIndex(dim, M, ef_construction) / CPHNSWIndex(const CPHNSWParams&)
 * (use sites evaluation/eval_sift.cpp:228, evaluation/test_gpu_build.cpp:155-162) and
 * GPUEncoder(dim, seed) (include/cphnsw/cuda/gpu_encoder.cuh:34).  Parameter bounds are those of
 * CPHNSWParams::finalize() (include/cphnsw/core/types.hpp:403-469).  Sign tables are generated
 * like RotationChain does (include/cphnsw/encoder/rotation.hpp:134-144,173-178). */
int cphnsw_b200_create(uint64_t dim, uint32_t K, uint32_t component_bytes, uint32_t M,
                       uint32_t ef_construction, uint64_t seed, int fht_convention, int device,
                       cphnsw_b200_index** out);
/* The same for the unified index's binary codes (CPHNSWIndex<K, 0>, include/cphnsw/api/index.hpp:71-90):
 * "binary_codes" is on from the start and a component is one byte whatever the dimension (it
 * holds a sign bit only). */
int cphnsw_b200_create_binary(uint64_t dim, uint32_t K, uint32_t M, uint32_t ef_construction, uint64_t seed,
                              int fht_convention, int device, cphnsw_b200_index** out);
int cphnsw_b200_destroy(cphnsw_b200_index* h);

/* Named tunables (CPHNSWParams fields, types.hpp:374-400, plus build/search knobs):
 *   "keep_pruned" (0/1, default 1), "profile" (0/1, see kernel_time),
 *   "prune" (0/1, default 1: the bulk build runs select_neighbors on the kNN candidates; 0 = the M nearest
 *            candidates are the links, build_with_gpu_knn(..., prune = false), evaluation/test_gpu_build.cpp:168-174),
 *   "knn_k" (candidates per node fed to select_neighbors, default min(2*M, 64)),
 *   "knn_kernel" (0 = pick, 1 = byte-wise distance, 2 = bit-sliced distance; K = 16/32/64 with uint8 codes or
 *                 in binary-code mode, K = 16/32 with uint16 codes of padded dim 1024, and one-byte binary codes of
 *                 any K <= 120 that is a multiple of 8, residual bits included when the primary part is one too),
 *   "search_kernel" (0 = pick: two warps per query whenever that kernel applies; 1 = one warp per query,
 *                    2 = two warps per query; the second needs
 *                    M <= 32, either K * padded_dim * 4 <= 32 KB or K <= 32, and a beam max(ef, k, rerank_k) of at most
 *                    1024 (2048 when K * padded_dim * 4 <= 32 KB); both return identical results),
 *   "binary_codes" (0/1, before any vector is added: 1 = the unified index's primary binary code
 *                   (include/cphnsw/core/codes.hpp:76-129 with R = 0): a component keeps only its sign bit, so
 *                   code distance = Hamming distance and the graph is built under it; search / search_and_rerank
 *                   walk under the Hamming distance to the query's code (unified search, include/cphnsw/api/index.hpp:177-214),
 *                   distances returned are Hamming distances (exact -<q,x> after a rerank); brute_force_search ranks by
 *                   Hamming distance; calibrate and search_multiprobe are not available.  Between build stages the
 *                   stored code of a node is its sign bits packed 32 per word (include/cphnsw/core/codes.hpp:21-52
 *                   packs 64 per word), which the walk compares by XOR and popcount; the array of one component per
 *                   bit exists only while add_batch_parallel / add_batch run; get_code, get_codes and the index file
 *                   still give one component per bit; get_param("stored_code_bytes") tells the bytes per node),
 *   "residual_bits" / "residual_shift" (binary-code mode only, before any vector is added: the unified index's
 *                   residual codes, ResidualCode<K, R> (include/cphnsw/core/codes.hpp:76-129).  The handle's K
 *                   counts primary + residual bits; the last residual_bits components are the residual bits (the
 *                   reference seeds its residual rotations seed + K_primary + r, i.e. rotations K_primary.. of one
 *                   chain) and every code distance becomes (h_primary << residual_shift) + h_residual
 *                   (include/cphnsw/core/types.hpp:284-302; shift 0..4).  (K - residual_bits) * component_bytes must
 *                   be a multiple of 4; the kNN graph runs on the bit-sliced kernel when K and K - residual_bits are
 *                   multiples of 8 and K <= 120, else on the byte-wise kernel),
 *   "build_seed" (0 = add_batch_parallel builds the exact code-distance kNN graph over everything, the
 *                 default; s > 0 = on an empty index only the first s vectors get the exact graph and
 *                 the others are inserted as add_batch does: O(n) instead of O(n^2) candidate search),
 *   "rank_prune" (0/1, default 0: the bulk build prunes the kNN lists by rank, see cphnsw_b200_rank_prune, instead of
 *                 running select_neighbors) and "rank_pruning_alpha" (1.0..3.0, default 1.1; CPHNSWParams::rank_pruning_alpha,
 *                 types.hpp:399-400,459-466),
 *   "exact_edges" (0/1, default 0: the bulk build chooses the links on the stored fp32 vectors instead of the codes - the
 *                 legacy "hybrid" construction, "True Cosine edges - the production path", evaluation/eval_master.cpp:251-272:
 *                 candidates of a node = its knn_k exact nearest neighbours by -<x,y> (the exact top-(knn_k+1) over all
 *                 vectors by (distance, id) with the node itself removed), then select_neighbors on those exact distances,
 *                 every distance summed in fp32 in d order; O(n^2 d) build, search unchanged; with "prune" = 0 the M exact
 *                 nearest are the links; incremental add_batch keeps choosing by code distance),
 *   "first_wait_polls" (0..2^22, default 2^22: polls granted to the FIRST bounded wait of a kNN-graph launch; a test
 *                 sets 0 to make that wait give up, which the call reports as CPHNSW_B200_E_DEVICE_WAIT),
 *   "entry_scan" (evenly spaced nodes scored for every query before the walk; default = k_entry),
 *   "k_entry" (1..100, default 4: how many of the scored nodes, the best, seed the walk). */
int cphnsw_b200_set_param(cphnsw_b200_index* h, const char* name, double value);
int cphnsw_b200_get_param(const cphnsw_b200_index* h, const char* name, double* value);

uint64_t cphnsw_b200_dim(const cphnsw_b200_index* h);
uint64_t cphnsw_b200_padded_dim(const cphnsw_b200_index* h);
uint64_t cphnsw_b200_size(const cphnsw_b200_index* h); /* CPHNSWIndex::size(), README.md:88 */

/* int8 [K][3][padded_dim] of +1/-1, the tables RandomHadamardRotation::get_signs() exposes
 * (include/cphnsw/encoder/rotation.hpp:116-121). set_ replaces them (e.g. tables drawn by
 * another standard library). */
int cphnsw_b200_get_sign_tables(const cphnsw_b200_index* h, int8_t* out);
int cphnsw_b200_set_sign_tables(cphnsw_b200_index* h, const int8_t* signs);

/* ---- stage entry points, host pointers ------------------------------------------------------ */

/* Replaces legacy CPEncoder<ComponentT,K>::encode / encode_batch
 * (include/cphnsw/encoder/cp_encoder.hpp:161-184,244-260) and GPUEncoder::encode_batch
 * (src/cuda/gpu_encoder.cu:430-471).  x float[n][dim] -> codes ComponentT[n][K]. */
int cphnsw_b200_encode(cphnsw_b200_index* h, const float* x, uint64_t n, void* codes_out);

/* Replaces legacy encode_query / GPUEncoder::encode_queries_batch (src/cuda/gpu_encoder.cu:473-513):
 * codes [nq][K]; rotated float[nq][K][padded_dim] (CPQuery::rotated_vecs, types.hpp:324-337) and
 * magnitudes float[nq][K] are optional (NULL to skip). */
int cphnsw_b200_encode_queries(cphnsw_b200_index* h, const float* q, uint64_t nq, void* codes_out,
                               float* rotated_out, float* magnitudes_out);

/* Replaces legacy hamming_distance(CPCode,CPCode) (use sites evaluation/debug_estimator.cpp:149,172):
 * out[na][nb] = number of differing components. */
int cphnsw_b200_code_distance(cphnsw_b200_index* h, const void* codes_a, uint64_t na,
                              const void* codes_b, uint64_t nb, uint16_t* out);

/* Replaces GPUKNNGraphBuilder::build (src/cuda/gpu_knn_graph.cu:330-415) with the CP-code metric:
 * rows [row_begin,row_end) against all n codes, self excluded, k smallest by (distance, id),
 * padded with 0xFFFFFFFF / 0xFFFF.  nbrs_out uint32[rows][k]; dist_out uint16[rows][k] or NULL. */
int cphnsw_b200_knn_graph(cphnsw_b200_index* h, const void* codes, uint64_t n, uint32_t k,
                          uint64_t row_begin, uint64_t row_end, uint32_t* nbrs_out, uint16_t* dist_out);

/* Replaces legacy select_neighbors (HNSW heuristic with keepPrunedConnections,
 * resources/hnsw-paper/consolidated.tex:93-115; flag types.hpp:390-391).
 * cand uint32[rows][k] in ascending (distance,id) order -> adj_out uint32[rows][M]. */
int cphnsw_b200_select_neighbors(cphnsw_b200_index* h, const void* codes, uint64_t n,
                                 const uint32_t* cand, uint32_t k, uint64_t row_begin, uint64_t row_end,
                                 uint32_t M, int keep_pruned, uint32_t* adj_out);

/* Rank-based pruning of kNN lists: the graph optimisation of CAGRA that the legacy index ran behind
 * build_with_gpu_knn(base, N, k, prune = true, alpha) (evaluation/test_gpu_build.cpp:168-174; parameter
 * "Detour threshold for rank-based pruning (CAGRA)", include/cphnsw/core/types.hpp:399-400).  The legacy source is
 * absent; the rule is the paper's (resources/arXiv-2308.15136v2/consolidated.tex:298-340), no distance involved:
 *   reorder  a route X -> Z -> Y (Z, Y in X's list, Y in Z's list) is a detour of the edge X -> Y when
 *            alpha * max(rank_X(Z), rank_Z(Y)) < rank_X(Y), ranks = 1-based list positions, compared in fp32
 *            (alpha = 1: the paper's condition); X keeps its M candidates with the fewest detours, ties by rank;
 *   reverse  P receives every X that kept P, ordered by (position of P in X's kept list, X);
 *   merge    kept list and reverse list of P are interleaved, kept list first, each id once, until M links are
 *            chosen; when one list runs out the other goes on alone.
 * cand uint32[n][k] (k <= 64) for ALL n nodes in ascending (distance, id) order -> adj_out uint32[n][M]. */
int cphnsw_b200_rank_prune(cphnsw_b200_index* h, const uint32_t* cand, uint64_t n, uint32_t k, uint32_t M, float alpha,
                           uint32_t* adj_out);

/* ---- index build and search, host pointers -------------------------------------------------- */

/* Replaces CPHNSWIndex::add_batch_parallel / add_batch (use sites evaluation/eval_master.cpp:89,
 * evaluation/eval_main.cpp:43): appends n vectors (ids continue from size()) and rebuilds the
 * graph over everything added so far: encode -> code-distance kNN graph (knn_k) -> select_neighbors. */
int cphnsw_b200_add_batch_parallel(cphnsw_b200_index* h, const float* x, uint64_t n);

/* Replaces CPHNSWIndex::add / add_batch (unified form include/cphnsw/api/index.hpp:98-164; legacy use
 * evaluation/qa_protocol.cpp:262): incremental insertion into the existing graph, batched.  The n
 * vectors are appended (ids continue from size()) in pieces no larger than the graph they join;
 * for every piece: encode; candidates of a new node = the 64 best of a walk of the EXISTING graph
 * under the code distance (beam ef_construction, seeds as for search; nodes of one piece do not see
 * each other); select_neighbors gives its M links; every old node chosen by new nodes re-selects
 * its row from (current row + the new nodes that chose it), the 64 closest by (distance, id).
 * On an empty index this is add_batch_parallel. */
int cphnsw_b200_add_batch(cphnsw_b200_index* h, const float* x, uint64_t n);

/* CPHNSWIndex::get_code (evaluation/debug_code_storage.cpp:75) for one node (ComponentT[K]) and for all nodes,
 * and the adjacency uint32[size][M] (FlatGraph neighbour ids, include/cphnsw/graph/flat_graph.hpp:179-181). */
int cphnsw_b200_get_code(const cphnsw_b200_index* h, uint32_t id, void* code_out);
int cphnsw_b200_get_codes(const cphnsw_b200_index* h, void* codes_out);
int cphnsw_b200_get_adjacency(const cphnsw_b200_index* h, uint32_t* adj_out);
/* ids scored for every query before the graph walk (entry_scan evenly spaced node ids); the k_entry best of
 * them seed the walk. */
int cphnsw_b200_get_entry_ids(const cphnsw_b200_index* h, uint32_t* ids_out, uint64_t* count);

/* Batched CPHNSWIndex::search(q,k,ef) (evaluation/eval_sift.cpp:387; engine
 * include/cphnsw/search/search_engine.hpp:86-193): graph walk under the asymmetric CP score,
 * ids uint32[nq][k], dists float[nq][k] ascending (negative scores), padded 0xFFFFFFFF / +inf.
 * Beam width is max(ef, k), at most 4096 (wider than 1024: the one-warp kernel).  stats (optional) uint32[nq][2] = expansions, distance evaluations. */
int cphnsw_b200_search_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k,
                             uint32_t ef, uint32_t* ids_out, float* dists_out, uint32_t* stats_out);

/* The same walk under the symmetric code distance to given query CODES (ComponentT[nq][K]): the unified index's
 * search, SearchEngine<Policy>::search over FlatGraph (include/cphnsw/search/search_engine.hpp:86-193) with
 * distance = code distance (Hamming distance in binary-code mode, residual weighting included); also the walk
 * search_multiprobe runs per probe code and add_batch runs per new node.  Distances are returned as floats. */
int cphnsw_b200_search_codes_batch(cphnsw_b200_index* h, const void* qcodes, uint64_t nq, uint32_t k, uint32_t ef,
                                   uint32_t* ids_out, float* dists_out, uint32_t* stats_out);

/* Batched CPHNSWIndex::search_and_rerank(q,k,ef,rerank_k) (evaluation/eval_master.cpp:145;
 * steps shown by hand at evaluation/eval_sift.cpp:539-563; replaces GPUBruteForce::rerank,
 * src/cuda/gpu_encoder.cu:605-664): beam max(ef, rerank_k), best rerank_k re-scored with
 * -<q,x> in fp32, sorted by (distance,id), best k returned. */
int cphnsw_b200_search_and_rerank_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k,
                                        uint32_t ef, uint32_t rerank_k, uint32_t* ids_out,
                                        float* dists_out, uint32_t* stats_out);

/* Batched CPHNSWIndex::search_multiprobe(q,k,ef,num_probes) (evaluation/eval_sift.cpp:430,469).  The legacy
 * source is absent; this follows the multiprobe scheme of the cross-polytope LSH paper
 * (resources/cross-polytope-lsh/consolidated.tex:391-425) on the data CPQuery keeps for it
 * (types.hpp:332-336): the num_probes (1..64) cheapest probe codes of the query are generated, the graph is
 * walked once per probe code under the symmetric code distance (beam max(ef,k), seeds as for search), and
 * the per-probe lists are merged: every node once with its smallest distance, ascending by (distance, id),
 * best k.  dists are code distances as floats.  num_probes * k <= 2048. */
int cphnsw_b200_search_multiprobe_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k,
                                        uint32_t ef, uint32_t num_probes, uint32_t* ids_out, float* dists_out);
/* Diagnostics the reference's evaluation programs call around the hot path.  The legacy sources
 * are absent; behaviour follows the call sites.
 *
 * Batched CPHNSWIndex::brute_force_search(q,k) (evaluation/eval_sift.cpp:283,329;
 * evaluation/test_k_variants.cpp:79): the k (<= 1024) nodes with the smallest asymmetric CP score
 * among all stored nodes, ascending by (score, id); no graph involved. */
int cphnsw_b200_brute_force_search_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k,
                                         uint32_t* ids_out, float* dists_out);
/* Exact search and rerank on fp32 vectors: GPUBruteForce (include/cphnsw/cuda/gpu_encoder.cuh:101-156;
 * src/cuda/gpu_encoder.cu:554-664) and the harness's compute_ground_truth
 * (evaluation/datasets/dataset_loader.hpp:187-212).  distance = -<q,x>, the dot product accumulated in
 * fp32 in d order; results ascending by (distance, id), rows padded with (CPHNSW_B200_INVALID_NODE, +inf);
 * k <= 128.  They run over the index's stored vectors unless set_exact_base gave others
 * (GPUBruteForce::set_base_vectors; float[n][dim] with the handle's dim, copied to the device; n = 0
 * drops them again).  rerank (GPUBruteForce::rerank): the k best of cand[nq][num_cand]; ids >= n and
 * CPHNSW_B200_INVALID_NODE are skipped. */
int cphnsw_b200_set_exact_base(cphnsw_b200_index* h, const float* base, uint64_t n);
int cphnsw_b200_exact_search_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k,
                                   uint32_t* ids_out, float* dists_out);
int cphnsw_b200_rerank_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, const uint32_t* cand,
                             uint32_t num_cand, uint32_t k, uint32_t* ids_out, float* dists_out);
/* CPHNSWIndex::verify_connectivity() (evaluation/eval_main.cpp:52, eval_sift.cpp:266): number of
 * nodes reachable from the entry nodes along the directed adjacency, entry nodes included. */
int cphnsw_b200_verify_connectivity(cphnsw_b200_index* h, uint64_t* reachable_out);
/* CPHNSWIndex::calibrate(num_samples, seed) (evaluation/eval_main.cpp:128-135, qa_protocol.cpp:263-270):
 * num_samples (1..65536) pairs (u,v) of stored nodes from std::mt19937_64(seed) (u = next() % n, then
 * v = next() % n); least-squares fit  -<x_u,x_v> ~ alpha * score(u,v) + beta  of the exact distance
 * against the asymmetric CP score, r_squared = squared correlation.  The fit is kept in the handle
 * (get_calibration) and used by search_calibrated. */
int cphnsw_b200_calibrate(cphnsw_b200_index* h, uint64_t num_samples, uint64_t seed, double* alpha_out,
                          double* beta_out, double* r_squared_out);
int cphnsw_b200_get_calibration(const cphnsw_b200_index* h, double* alpha_out, double* beta_out,
                                double* r_squared_out, uint64_t* num_samples_out);
/* Batched CPHNSWIndex::search_calibrated(q,k,ef) and search_calibrated_and_rerank(q,k,ef,rerank_k)
 * (evaluation/eval_main.cpp:170,189): the walk of search / search_and_rerank; with rerank_k == 0
 * the returned distances are alpha * score + beta (an estimate of the exact distance; alpha > 0
 * keeps the order), with rerank_k > 0 they are the exact reranked distances. */
int cphnsw_b200_search_calibrated_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k,
                                        uint32_t ef, uint32_t rerank_k, uint32_t* ids_out, float* dists_out);

/* Sign bits of all stored codes packed like the unified index's ResidualCode<K,0>::primary
 * (include/cphnsw/core/codes.hpp:21-52): uint64[size][(K+63)/64], bit r of a row = 1 iff the winning
 * coordinate of rotation r is negative.  Works in both code modes (it is bit 0 of every component). */
int cphnsw_b200_get_binary_codes(const cphnsw_b200_index* h, uint64_t* words_out);

/* Index file (the reference has no save/load; its rotation.hpp get_signs() exists "for serialization" only).  One little-endian file: magic "CPHNSWB2", format version, the constructor
 * arguments, the tunables, the calibration, then sign tables int8[K][3][padded_dim], vectors
 * float[n][dim], codes ComponentT[n][K], adjacency uint32[n][M].  load creates a new handle on `device`
 * holding exactly the saved index (no re-encoding, no graph rebuild); it can be searched at once and
 * extended with add_batch_parallel. */
int cphnsw_b200_save(cphnsw_b200_index* h, const char* path);
int cphnsw_b200_load(const char* path, int device, cphnsw_b200_index** out);

/* The probe codes themselves, ComponentT[nq][num_probes][K], primary code first (legacy multiprobe.hpp). */
int cphnsw_b200_probe_codes(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t num_probes,
                            void* codes_out);

/* ---- device-pointer variants (inputs already resident in HBM; used for sharded builds) ------- */

int cphnsw_b200_encode_dev(cphnsw_b200_index* h, const float* d_x, uint64_t n, void* d_codes,
                           float* d_rotated, float* d_magnitudes, void* stream);
int cphnsw_b200_code_distance_dev(cphnsw_b200_index* h, const void* d_a, uint64_t na, const void* d_b,
                                  uint64_t nb, uint16_t* d_out, void* stream);
int cphnsw_b200_knn_graph_dev(cphnsw_b200_index* h, const void* d_codes, uint64_t n, uint32_t k,
                              uint64_t row_begin, uint64_t row_end, uint32_t* d_nbrs, uint16_t* d_dist,
                              void* stream);
int cphnsw_b200_select_neighbors_dev(cphnsw_b200_index* h, const void* d_codes, uint64_t n,
                                     const uint32_t* d_cand, uint32_t k, uint64_t row_begin,
                                     uint64_t row_end, uint32_t M, int keep_pruned, uint32_t* d_adj,
                                     void* stream);
/* Install a complete index from device buffers (copied, not retained): vectors float[n][dim],
 * codes [n][K], adjacency uint32[n][M].  Used after a sharded build has all-gathered its rows.
 * The rows are taken as they are: an id that names no node (>= n) is treated as CPHNSW_B200_INVALID_NODE
 * by every kernel that reads the adjacency (search, connectivity, the reverse-edge pass of add_batch),
 * never dereferenced.  The same holds for candidate ids given to select_neighbors and for loaded files. */
int cphnsw_b200_install_dev(cphnsw_b200_index* h, const float* d_vectors, const void* d_codes,
                            const uint32_t* d_adj, uint64_t n, void* stream);
/* The same from host buffers (FlatGraph::add_node + add_neighbor for every node,
 * include/cphnsw/graph/flat_graph.hpp:80-98,204-208). */
int cphnsw_b200_install(cphnsw_b200_index* h, const float* vectors, const void* codes, const uint32_t* adj, uint64_t n);
/* The two halves of cphnsw_b200_rank_prune for row-block sharded builds: reorder writes the M kept ids of rows
 * [row_begin, row_end) from the candidate lists of ALL n nodes; merge needs the kept rows of all n nodes (gathered
 * in between) and writes the final rows of the range. */
int cphnsw_b200_rank_reorder_dev(cphnsw_b200_index* h, const uint32_t* d_cand, uint64_t n, uint32_t k, uint64_t row_begin,
                                 uint64_t row_end, uint32_t M, float alpha, uint32_t* d_kept, void* stream);
int cphnsw_b200_rank_merge_dev(cphnsw_b200_index* h, const uint32_t* d_kept, uint64_t n, uint32_t M, uint64_t row_begin,
                               uint64_t row_end, uint32_t* d_adj, void* stream);
/* d_q float[nq][dim]; outputs device uint32[nq][k] / float[nq][k]; rerank_k = 0 means plain search. */
int cphnsw_b200_search_dev(cphnsw_b200_index* h, const float* d_q, uint64_t nq, uint32_t k, uint32_t ef,
                           uint32_t rerank_k, uint32_t* d_ids, float* d_dists, uint32_t* d_stats,
                           void* stream);
/* exact_search over d_base float[n][dim] (device) for d_q float[nq][dim]; outputs device uint32[nq][k] / float[nq][k]. */
int cphnsw_b200_exact_search_dev(cphnsw_b200_index* h, const float* d_base, uint64_t n, const float* d_q,
                                 uint64_t nq, uint32_t k, uint32_t* d_ids, float* d_dists, void* stream);
/* ---- one index over several GPUs of one box -------------------------------------------------------------
 * The reference is single-device (BuildParams::gpu_device is declared and never read, include/cphnsw/api/config.hpp:55-56);
 * this is the multi-GPU form of the same calls: one process, one replica of the index per device.
 * add_batch_parallel shards the rows into contiguous blocks: every device encodes its block, the codes are
 * all-gathered with NCCL, every device computes the kNN rows and the pruned rows of its block against all codes, the
 * adjacency and vector blocks are all-gathered and every device installs the complete index - the adjacency is the
 * one a single device builds, bit for bit.  search splits the query batch across the replicas (batches smaller than
 * 32 queries per device go to one replica whole, successive calls going round the replicas, so that single-query
 * calls from many host threads use all devices).  n_gpus = 0 takes every usable device; devices = NULL means
 * ordinals 0..n_gpus-1.  NCCL (libnccl.so.2) is loaded at run time, and only when n_gpus > 1.
 * Thread safety is that of the plain handle: searches from any number of threads, builds exclude one another. */
typedef struct cphnsw_b200_sharded cphnsw_b200_sharded;
int cphnsw_b200_sharded_create(uint64_t dim, uint32_t K, uint32_t component_bytes, uint32_t M, uint32_t ef_construction,
                               uint64_t seed, int fht_convention, int binary_codes, int n_gpus, const int* devices,
                               cphnsw_b200_sharded** out);
/* a saved index (cphnsw_b200_save) loaded onto every device */
int cphnsw_b200_sharded_load(const char* path, int n_gpus, const int* devices, cphnsw_b200_sharded** out);
int cphnsw_b200_sharded_destroy(cphnsw_b200_sharded* s);
int cphnsw_b200_sharded_gpus(const cphnsw_b200_sharded* s);
uint64_t cphnsw_b200_sharded_size(const cphnsw_b200_sharded* s);
/* The replica on the g-th device: an ordinary handle, owned by the sharded index.  Read-only calls (get_codes,
 * get_adjacency, save, verify_connectivity, the stage calls) may use any replica; calls that change a handle must be
 * made on every replica alike (set_param and the add calls below do that). */
cphnsw_b200_index* cphnsw_b200_sharded_replica(const cphnsw_b200_sharded* s, int g);
int cphnsw_b200_sharded_set_param(cphnsw_b200_sharded* s, const char* name, double value);
/* CPHNSWIndex::add_batch_parallel over all devices (an index that already holds nodes, a seeded build or fewer than
 * 64 rows per device: every replica runs the whole call instead) and add_batch (every replica inserts the same rows). */
int cphnsw_b200_sharded_add_batch_parallel(cphnsw_b200_sharded* s, const float* x, uint64_t n);
int cphnsw_b200_sharded_add_batch(cphnsw_b200_sharded* s, const float* x, uint64_t n);
/* The batched searches over all replicas.  mode: 0 search_batch, 1 search_and_rerank_batch (arg = rerank_k),
 * 2 search_multiprobe_batch (arg = num_probes), 3 brute_force_search_batch, 4 search_calibrated_batch (arg = rerank_k);
 * arguments and outputs as in the call of that name (stats_out: modes 0 and 1, else NULL). */
int cphnsw_b200_sharded_search(cphnsw_b200_sharded* s, int mode, const float* q, uint64_t nq, uint32_t k, uint32_t ef,
                               uint32_t arg, uint32_t* ids_out, float* dists_out, uint32_t* stats_out);
/* Host-clock milliseconds of the stages of the last sharded build: encode (with the upload), all-gather of codes,
 * kNN rows, pruning, all-gather of adjacency and vectors, installation.  ms_out double[CPHNSW_B200_SHARDED_STAGES]. */
#define CPHNSW_B200_SHARDED_STAGES 6
int cphnsw_b200_sharded_stage_times(const cphnsw_b200_sharded* s, double* ms_out);

/* Code distance for callers that cannot allocate device memory.  No counterpart in the reference.
 *
 * Some hosts of this library run under a fixed memory plan: a serving process whose device memory
 * was carved up at start-up, a plugin running inside another framework's allocator, or code on a
 * latency path where cudaMalloc's implicit device synchronisation is not acceptable.  The ordinary
 * entry points grow scratch buffers with cudaMalloc on demand; this one never allocates or frees
 * anything (no cudaMalloc, cudaFree or allocating library routine).  It needs no index handle either
 * (creating one allocates): it works on the CURRENT CUDA device and takes the code shape directly.
 *
 * Same result as cphnsw_b200_code_distance_dev: d_out[na][nb] = number of differing components
 * between code rows d_a[na][K] and d_b[nb][K] (device pointers, caller-owned, asynchronous on `stream`).
 * The padded copies of both operands that the kernel reads are kept in a 1 MiB array built into the
 * library's device image (every GPU that loads the library holds it until the process exits), hence
 * the limit: (na + nb) * R <= 1 MiB, where R is the row size K*component_bytes rounded up to 16, 32,
 * 64 or 128 bytes (32,768 rows at K=32 uint8).  Larger inputs are rejected with CPHNSW_B200_E_INVALID.
 *
 * The first call on each device looks up the array's device address; make that first call outside
 * any stream capture.  All calls share the one array: it is fully rewritten by each call (nothing
 * from an earlier call is read), but two calls whose kernels can overlap on the GPU - different
 * streams, or different threads - race on it; serialise them.
 *
 * The plain count only: the residual weighting of a binary-code index ("residual_bits", "residual_shift") belongs
 * to a handle and is not applied here. */
int cphnsw_b200_code_distance_noalloc(const void* d_a, uint64_t na, const void* d_b, uint64_t nb, uint32_t K,
                                      uint32_t component_bytes, uint16_t* d_out, void* stream);

/* Reads and clears the device-side status word the kernels raise when a bounded wait runs out. */
int cphnsw_b200_check_device_status(cphnsw_b200_index* h);

/* Kernel timing for benchmarks (no counterpart in the reference, which times with a host clock,
 * evaluation/metrics/recall.hpp:109-130).  With set_param("profile", 1) every launch of a kernel
 * family is bracketed by CUDA events on its stream; this call waits for them, returns the summed
 * device time and the number of launches since the last call, and resets the family's record.
 * kind: 0 encode, 1 code distance, 2 kNN graph, 3 select_neighbors, 4 search. */
int cphnsw_b200_kernel_time(cphnsw_b200_index* h, int kind, double* total_ms, uint64_t* launches);

/* Number of kernel launches issued through this handle so far (for benchmark accounting). */
uint64_t cphnsw_b200_launch_count(const cphnsw_b200_index* h);

#ifdef __cplusplus
}
#endif
#endif /* CPHNSW_B200_H */
