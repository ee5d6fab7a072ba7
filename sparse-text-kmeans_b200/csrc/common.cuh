// Shared declarations of the cphnsw_b200 library: the index handle, error plumbing and the
// launcher prototypes of each kernel family.  sm_100a only.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <vector>

#include "../../include/cphnsw_b200.h"

namespace cpb {

constexpr uint32_t kInvalidNode = 0xFFFFFFFFu;

// Device-side status word values raised by kernels (read with cphnsw_b200_check_device_status).
constexpr uint32_t kStatusOk = 0;
constexpr uint32_t kStatusWaitTimeout = 1;  // a bounded mbarrier wait ran out

void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define CPB_CUDA(expr)                                        \
    do {                                                      \
        cudaError_t e__ = (expr);                             \
        if (e__ != cudaSuccess) return cpb::cuda_fail(e__, #expr); \
    } while (0)

#define CPB_TRY(expr)             \
    do {                          \
        int rc__ = (expr);        \
        if (rc__ != 0) return rc__; \
    } while (0)

// Lets a kernel use as much dynamic shared memory as the device grants a block.  The attribute belongs to the
// function, not to the launch: concurrent callers that each set "what my launch needs" would lower it under one
// another's feet, so every caller sets the same, largest value (the device's opt-in limit less the kernel's static
// shared memory).
template <class F>
inline cudaError_t allow_max_dynamic_smem(F* kernel) {
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, kernel);
    if (e != cudaSuccess) return e;
    int dev = 0, optin = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return e;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - int(fa.sharedSizeBytes));
}

// kernel families whose launches can be timed
enum KernelKind { kKernelEncode = 0, kKernelCodeDistance = 1, kKernelKnn = 2, kKernelSelect = 3, kKernelSearch = 4 };
constexpr int kKernelKinds = 5;
struct EventPair {
    cudaEvent_t start = nullptr, stop = nullptr;
};

// RAII device buffer (the library owns every scratch / index allocation through this).
struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
    DevBuf() = default;
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    ~DevBuf() { release(); }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        bytes = 0;
    }
    // grow-only; contents are not preserved
    int reserve(size_t n) {
        if (n <= bytes && p) return 0;
        release();
        if (n == 0) n = 16;
        CPB_CUDA(cudaMalloc(&p, n));
        bytes = n;
        return 0;
    }
    void swap(DevBuf& o) {
        void* tp = p;
        size_t tb = bytes;
        p = o.p, bytes = o.bytes;
        o.p = tp, o.bytes = tb;
    }
    template <class T>
    T* as() const { return reinterpret_cast<T*>(p); }
};

// Everything one search call writes besides its outputs: a stream, the staging and result buffers, the
// work counter and the visited slots of its launch.  A handle keeps a pool of these so that search calls from
// several host threads run side by side (the reference's callers search from OpenMP loops,
// evaluation/eval_sift.cpp:380-387).  `wide` contexts own visited slots for a launch that fills the GPU,
// narrow ones for launches of up to kNarrowQueries queries, one block per query.
constexpr uint32_t kNarrowQueries = 32;
// widest beam of a search: the one-warp kernel keeps W as one sorted array of up to this many members in shared
// memory (32 KB at 4,096); the two-warp kernel's tiered W holds 1,024 and is used up to that width
constexpr uint32_t kMaxBeam = 4096;
struct SearchCtx {
    cudaStream_t stream = nullptr;
    cudaEvent_t done = nullptr;  // recorded behind the last work that used this scratch on a caller's stream
    bool pending = false;        // `done` has to be waited for before the scratch is reused
    bool busy = false;
    bool wide = false;
    DevBuf d_visited, d_epochs, d_counter;
    uint64_t vis_stride = 0;
    size_t vis_slots = 0;
    DevBuf d_qtables, d_qcodes, d_q, d_out_ids, d_out_dist, d_stats;
    DevBuf d_probe_codes, d_probe_ids, d_probe_dist;  // search_multiprobe
    ~SearchCtx() {
        if (done) cudaEventDestroy(done);
        if (stream) cudaStreamDestroy(stream);
    }
};

}  // namespace cpb

struct cphnsw_b200_index {
    // parameters (CPHNSWParams, include/cphnsw/core/types.hpp:374-400)
    uint64_t dim = 0, P = 0;
    uint32_t K = 0, comp_bytes = 0, M = 0, ef_construction = 0;
    uint64_t seed = 42;
    int convention = CPHNSW_B200_FHT_AVX512;
    int device = 0;
    int keep_pruned = 1;
    int prune = 1;  // 0: the bulk build keeps the M nearest kNN candidates instead of running select_neighbors
    uint32_t k_entry = 4, knn_k = 0, entry_scan = 0;
    int knn_kernel = 0;  // 0 = pick, 1 = byte-wise distance, 2 = bit-sliced distance
    int search_kernel = 0;  // 0 = pick, 1 = one warp per query, 2 = two warps per query
    int search_table_smem = 1;  // 0: the query table is read in place even when it would fit shared memory
    int binary_codes = 0;  // 1: components keep only the sign bit (Hamming metric), search walks under the code distance
    // residual codes of the binary mode: the last residual_bits components are residual bits, a primary mismatch
    // counts 2^residual_shift (combined distance (h_p << shift) + h_r, include/cphnsw/core/types.hpp:284-302)
    uint32_t residual_bits = 0, residual_shift = 0;
    uint32_t build_seed = 0;  // 0: add_batch_parallel builds the exact kNN graph; else only of this many nodes, the rest inserted
    int sm_count = 0;
    // polls the kNN kernels grant their FIRST tile wait ("first_wait_polls"; every other wait keeps the full
    // limit).  0 makes that wait give up at once: the way a test reaches the lost-wait path.
    uint32_t first_wait_polls = 1u << 22;
    int exact_edges = 0;              // bulk build picks candidates and links on the fp32 vectors (legacy hybrid construction)
    int rank_prune = 0;               // bulk build prunes by detourable-route count instead of select_neighbors
    float rank_pruning_alpha = 1.1f;  // CPHNSWParams::rank_pruning_alpha (include/cphnsw/core/types.hpp:399-400)

    std::vector<int8_t> signs;  // host [K][3][P]
    cpb::DevBuf d_signs;        // float [K][3][P], +-1 with the FHT convention folded into layers 1,2
    cpb::DevBuf d_signbits;     // padded dim 1024 only: the same diagonals bit-packed, uint32 [K][3][32]
    // uint32 words: 0 status of bounded device waits, 1 query counter of a search launch, 2 "an adjacency
    // row repeats an id", 4-5 frontier sizes of the connectivity BFS, 6-7 counters of the reverse-edge pass
    cpb::DevBuf d_status;

    // index contents
    uint64_t n = 0;
    cpb::DevBuf d_vectors, d_codes, d_adj, d_entry, d_entry_codes;
    cpb::DevBuf d_packed;       // binary-code mode: the sign bits of every node packed 32 per word, uint32 [n][packed_words],
    int packed_words = 0;       // which is what the walk reads (popcount of an XOR); 0 outside that mode
    bool codes_released = false;  // binary-code mode between build stages: d_codes is freed, the packed bits are the stored
                                  // code (8 times smaller); stages that need one byte per bit unpack them first
    cpb::DevBuf d_exact_base;  // vectors given to set_exact_base (exact_search / rerank run over them instead of d_vectors)
    uint64_t n_exact = 0;
    uint32_t n_entry = 0;
    int adj_rows_distinct = 0;  // no adjacency row lists a node twice (scan_adjacency_rows)
    // calibrate(): true distance ~ alpha * CP score + beta (identity until calibrate is called)
    double calib_alpha = 1.0, calib_beta = 0.0, calib_r2 = 0.0;
    uint64_t calib_samples = 0;

    // Locking: search* calls hold `rw` shared and work in a SearchCtx of their own; every call that changes the
    // index or uses the stage scratch below holds it exclusively.
    mutable std::shared_mutex rw;
    std::mutex ctx_mu;
    std::condition_variable ctx_cv;
    std::vector<std::unique_ptr<cpb::SearchCtx>> ctxs;
    // scratch of calibrate / encode_queries (rotated vectors)
    cpb::DevBuf d_qtables, d_qcodes, d_q;
    // stage scratch for the host-pointer entry points
    cpb::DevBuf s_in, s_in2, s_out, s_out2, s_pad, s_pad2, s_sliced;
    cpb::DevBuf s_rank, s_kept;  // rank-based pruning: reverse lists, kept rows

    std::atomic<uint64_t> launches{0};

    // optional kernel timing ("profile" parameter): CUDA event pairs recorded around launches
    int profile = 0;
    std::mutex ev_mu;
    std::vector<cpb::EventPair> events[cpb::kKernelKinds];
    size_t events_used[cpb::kKernelKinds] = {0, 0, 0, 0, 0};
    ~cphnsw_b200_index();
};

namespace cpb {

// padded code row width (32-bit words) used by the distance kernels: 4, 8, 16 or 32; 0 = unsupported
int code_row_words(uint32_t K, uint32_t comp_bytes);

// ---- launchers (each returns 0 or a negative status and counts its launches in h) ----
int launch_encode(cphnsw_b200_index* h, const float* d_x, uint64_t n, void* d_codes, float* d_rot,
                  float* d_mag, cudaStream_t st);
int launch_code_distance(cphnsw_b200_index* h, const void* d_a, uint64_t na, const void* d_b,
                         uint64_t nb, uint16_t* d_out, cudaStream_t st);
int launch_knn_graph(cphnsw_b200_index* h, const void* d_codes, uint64_t n, uint32_t k, uint64_t row_begin,
                     uint64_t row_end, uint32_t* d_nbrs, uint16_t* d_dist, cudaStream_t st);
// bit-sliced variant of the kNN kernel (uint8 components, K = 16 or 32)
bool knn_sliced_supported(const cphnsw_b200_index* h);
int launch_knn_graph_sliced(cphnsw_b200_index* h, const void* d_codes, uint64_t n, uint32_t k, uint64_t row_begin,
                            uint64_t row_end, uint32_t* d_nbrs, uint16_t* d_dist, cudaStream_t st);
int launch_select_neighbors(cphnsw_b200_index* h, const void* d_codes, uint64_t n, const uint32_t* d_cand,
                            uint32_t k, uint64_t row_begin, uint64_t row_end, uint32_t M, int keep_pruned,
                            uint32_t* d_adj, cudaStream_t st, const uint32_t* d_row_ids = nullptr);
// rank-based pruning of kNN lists (rank_prune.cu): d_cand uint32[n][k] for ALL n nodes; reorder writes the M kept
// ids of rows [row_begin, row_end); merge needs the kept rows of all n nodes and writes the final rows of the range
int launch_rank_reorder(cphnsw_b200_index* h, uint64_t n, const uint32_t* d_cand, uint32_t k, uint64_t row_begin,
                        uint64_t row_end, uint32_t M, float alpha, uint32_t* d_kept, cudaStream_t st);
int launch_rank_merge(cphnsw_b200_index* h, uint64_t n, const uint32_t* d_kept, uint32_t M, uint64_t row_begin,
                      uint64_t row_end, uint32_t* d_adj, cudaStream_t st);
int launch_rank_prune(cphnsw_b200_index* h, uint64_t n, const uint32_t* d_cand, uint32_t k, uint32_t M, float alpha,
                      uint32_t* d_adj, cudaStream_t st);
// links chosen on the fp32 vectors (exact_edges.cu): exact nearest neighbours as candidates, select_neighbors on exact distances
int launch_exact_candidates(cphnsw_b200_index* h, const float* d_vectors, uint64_t n, uint32_t k, uint64_t row_begin,
                            uint64_t row_end, uint32_t* d_cand, cudaStream_t st);
int launch_select_exact(cphnsw_b200_index* h, const float* d_vectors, uint64_t n, const uint32_t* d_cand, uint32_t k,
                        uint64_t row_begin, uint64_t row_end, uint32_t M, int keep_pruned, uint32_t* d_adj, cudaStream_t st);
// incremental insertion: old nodes chosen by the new rows [n_old, n_old + m) of d_adj re-select their rows
int launch_reverse_edges(cphnsw_b200_index* h, const void* d_codes, uint64_t n_old, uint64_t m, uint32_t* d_adj,
                         uint32_t M, int keep_pruned, cudaStream_t st);
int launch_search(cphnsw_b200_index* h, SearchCtx& cx, const float* d_q, const float* d_tables, uint64_t nq, uint32_t k,
                  uint32_t beam, uint32_t rerank_k, uint32_t* d_ids, float* d_dists, uint32_t* d_stats,
                  cudaStream_t st, const void* d_qcodes = nullptr, int scan_only = 0);
int gather_rows(cphnsw_b200_index* h, const void* src, size_t row_bytes, const uint32_t* d_ids, uint32_t n_ids, void* dst,
                cudaStream_t st);
// diagnostics (diagnostics.cu)
int launch_connectivity(cphnsw_b200_index* h, uint64_t* reachable, cudaStream_t st);
int launch_calibration_samples(cphnsw_b200_index* h, const float* d_tables, const uint32_t* d_u, const uint32_t* d_v,
                               uint32_t m, float* d_x, float* d_y, cudaStream_t st);
int launch_affine(cphnsw_b200_index* h, float* d_dist, uint64_t n, float alpha, float beta, cudaStream_t st);
int launch_pack_sign_bits(cphnsw_b200_index* h, const void* d_codes, uint64_t n, uint64_t* d_out, cudaStream_t st);
// exact inner-product top-k and rerank over fp32 vectors (exact.cu)
int launch_exact_search(cphnsw_b200_index* h, const float* d_base, uint64_t n, const float* d_q, uint64_t nq, uint32_t k,
                        uint32_t* d_ids, float* d_dist, cudaStream_t st);
int launch_rerank(cphnsw_b200_index* h, const float* d_base, uint64_t n, const float* d_q, uint64_t nq, const uint32_t* d_cand,
                  uint32_t num_cand, uint32_t k, uint32_t* d_ids, float* d_dist, cudaStream_t st);
// multiprobe sequence of rotated queries [nq][K][P] -> probe codes [nq][T][K]; merge of per-probe results
int launch_probe_codes(cphnsw_b200_index* h, const float* d_rotated, uint64_t nq, uint32_t T, void* d_out,
                       cudaStream_t st);
int launch_merge_probes(cphnsw_b200_index* h, const uint32_t* d_ids, const float* d_dist, uint64_t nq, uint32_t T,
                        uint32_t k, uint32_t* d_out_ids, float* d_out_dist, cudaStream_t st);
// visited slots and epoch counters of a context for an index of n nodes
int prepare_search_scratch(cphnsw_b200_index* h, SearchCtx& cx, cudaStream_t st);
// after n changed: every context's visited array is dropped (sized by n)
void drop_search_scratch(cphnsw_b200_index* h);
// looks for adjacency rows that list a node twice and sets h->adj_rows_distinct (after d_adj changes)
int scan_adjacency_rows(cphnsw_b200_index* h, cudaStream_t st);
// copies the codes of the entry ids into one contiguous buffer (after d_entry / d_codes change)
int gather_entry_codes(cphnsw_b200_index* h, cudaStream_t st);
// binary-code mode: d_codes rebuilt from the packed bits if it was released (callers hold the handle exclusively)
int ensure_codes(cphnsw_b200_index* h, cudaStream_t st);

// Brackets one kernel launch with an event pair when profiling is on (no-ops otherwise).
struct LaunchTimer {
    cphnsw_b200_index* h;
    int kind;
    cudaStream_t st;
    EventPair* ev = nullptr;
    LaunchTimer(cphnsw_b200_index* h_, int kind_, cudaStream_t st_);
    ~LaunchTimer();
};

}  // namespace cpb
