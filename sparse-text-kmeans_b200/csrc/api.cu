// C ABI of cphnsw_b200: handle lifetime, parameter validation, host<->device staging and the
// build / search orchestration on top of the kernel launchers.  No CPU implementation of any
// stage lives here: without a usable sm_100 device every call fails.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <random>

#include "common.cuh"

namespace cpb {

static thread_local std::string g_error;

void set_error(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) in %s", int(e), cudaGetErrorString(e), what);
    return CPHNSW_B200_E_CUDA;
}

LaunchTimer::LaunchTimer(cphnsw_b200_index* h_, int kind_, cudaStream_t st_) : h(h_), kind(kind_), st(st_) {
    if (!h->profile) return;
    std::lock_guard<std::mutex> lock(h->ev_mu);
    auto& pool = h->events[kind];
    size_t& used = h->events_used[kind];
    if (used == pool.size()) {
        if (pool.size() == pool.capacity()) return;  // growing would move the pairs other timers point at
        EventPair e;
        if (cudaEventCreate(&e.start) != cudaSuccess || cudaEventCreate(&e.stop) != cudaSuccess) return;
        pool.push_back(e);
    }
    ev = &pool[used++];
    cudaEventRecord(ev->start, st);
}
LaunchTimer::~LaunchTimer() {
    if (ev) cudaEventRecord(ev->stop, st);
}

namespace {

uint64_t next_pow2(uint64_t n) {
    uint64_t p = 1;
    while (p < n) p *= 2;
    return p;
}

// +-1 float tables for the device: layer 0 as drawn; layers 1 and 2 multiplied by the diagonal
// the reference's SIMD FHT leaves on its output (element i negated when popcount(i & (W-1)) is
// odd; W = 16 for an AVX-512 build at P >= 16, 8 for AVX2 at P >= 8, none for scalar —
// include/cphnsw/encoder/transform/fht.hpp:81-87,141-147).
int upload_signs(cphnsw_b200_index* h) {
    const size_t P = h->P, K = h->K;
    size_t w = 1;
    if (h->convention == CPHNSW_B200_FHT_AVX512 && P >= 16) w = 16;
    else if (h->convention >= CPHNSW_B200_FHT_AVX2 && P >= 8) w = 8;
    std::vector<float> f(K * 3 * P);
    for (size_t r = 0; r < K; ++r)
        for (size_t l = 0; l < 3; ++l)
            for (size_t i = 0; i < P; ++i) {
                float s = float(h->signs[(r * 3 + l) * P + i]);
                if (l > 0 && (__builtin_popcountll(i & (w - 1)) & 1)) s = -s;
                f[(r * 3 + l) * P + i] = s;
            }
    CPB_TRY(h->d_signs.reserve(f.size() * sizeof(float)));
    CPB_CUDA(cudaMemcpy(h->d_signs.p, f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice));
    if (P == 1024) {
        // bit-packed copy for the 1024-point kernel (a set bit negates): layer 0 in the consecutive
        // layout (word w, bit b <-> element 32*w + b), layers 1 and 2 in the column layout
        // (word l, bit j <-> element 32*j + l)
        std::vector<uint32_t> bits(K * 3 * 32, 0u);
        for (size_t r = 0; r < K; ++r)
            for (size_t l = 0; l < 3; ++l)
                for (size_t i = 0; i < P; ++i)
                    if (f[(r * 3 + l) * P + i] < 0.0f) {
                        if (l == 0) bits[(r * 3 + l) * 32 + i / 32] |= 1u << (i % 32);
                        else bits[(r * 3 + l) * 32 + i % 32] |= 1u << (i / 32);
                    }
        CPB_TRY(h->d_signbits.reserve(bits.size() * 4));
        CPB_CUDA(cudaMemcpy(h->d_signbits.p, bits.data(), bits.size() * 4, cudaMemcpyHostToDevice));
    }
    return 0;
}

int bind(const cphnsw_b200_index* h) {
    if (!h) {
        set_error("null index handle");
        return CPHNSW_B200_E_INVALID;
    }
    CPB_CUDA(cudaSetDevice(h->device));
    return 0;
}

int check_status(cphnsw_b200_index* h) {
    uint32_t s = 0;
    CPB_CUDA(cudaMemcpy(&s, h->d_status.p, 4, cudaMemcpyDeviceToHost));
    if (s != kStatusOk) {
        CPB_CUDA(cudaMemset(h->d_status.p, 0, 4));
        set_error("a bounded device-side wait ran out (status %u); results of the last call are invalid", s);
        return CPHNSW_B200_E_DEVICE_WAIT;
    }
    return 0;
}

size_t code_row_bytes(const cphnsw_b200_index* h) { return size_t(h->K) * h->comp_bytes; }

int set_entry_ids(cphnsw_b200_index* h) {
    uint64_t s = h->entry_scan ? h->entry_scan : h->k_entry;
    if (s > h->n) s = h->n;
    std::vector<uint32_t> ids(s);
    for (uint64_t i = 0; i < s; ++i) ids[i] = uint32_t((unsigned __int128)i * h->n / s);
    h->n_entry = uint32_t(s);
    CPB_TRY(h->d_entry.reserve(s * 4 + 16));
    if (s) CPB_CUDA(cudaMemcpy(h->d_entry.p, ids.data(), s * 4, cudaMemcpyHostToDevice));
    CPB_TRY(gather_entry_codes(h, 0));
    CPB_TRY(scan_adjacency_rows(h, 0));
    CPB_CUDA(cudaStreamSynchronize(0));
    if (h->binary_codes && h->packed_words) {
        // binary-code mode: from here on the packed sign bits are the stored code (the walk reads them, and so do the
        // accessors); the array of one byte per bit comes back when a build stage needs it (ensure_codes)
        h->d_codes.release();
        h->codes_released = true;
    }
    return 0;
}

// the stored codes of binary-code mode, one component per bit, rebuilt on the host from the packed bits
// (accessors that hold the handle shared and may not touch its device buffers)
int host_codes_from_packed(const cphnsw_b200_index* h, uint64_t first, uint64_t count, unsigned char* out) {
    if (count == 0) return 0;
    const size_t words = size_t(h->packed_words);
    std::vector<uint32_t> w(count * words);
    CPB_CUDA(cudaMemcpy(w.data(), h->d_packed.as<uint32_t>() + first * words, w.size() * 4, cudaMemcpyDeviceToHost));
    const size_t cb = h->comp_bytes, K = h->K;
    std::memset(out, 0, count * K * cb);
    for (uint64_t i = 0; i < count; ++i)
        for (size_t r = 0; r < K; ++r) out[(i * K + r) * cb] = (unsigned char)((w[i * words + (r >> 5)] >> (r & 31)) & 1u);
    return 0;
}

// grows a device buffer to new_bytes keeping its first keep_bytes
int grow_keep(DevBuf& b, size_t keep_bytes, size_t new_bytes) {
    if (b.p && new_bytes <= b.bytes) return 0;
    void* p = nullptr;
    const size_t cap = new_bytes + new_bytes / 2;
    CPB_CUDA(cudaMalloc(&p, cap));
    if (b.p && keep_bytes) {
        cudaError_t e = cudaMemcpy(p, b.p, keep_bytes, cudaMemcpyDeviceToDevice);
        if (e != cudaSuccess) {
            cudaFree(p);
            CPB_CUDA(e);
        }
    }
    b.release();
    b.p = p;
    b.bytes = cap;
    return 0;
}

// adjacency of the first n nodes (codes in d_codes) into `adj`: kNN candidates, then pruning.  The
// handle's own adjacency and node count are left alone; the caller commits them on success.
int build_graph(cphnsw_b200_index* h, uint64_t n, DevBuf& adj, cudaStream_t st) {
    uint32_t k = h->knn_k ? h->knn_k : (2 * h->M < 64 ? 2 * h->M : 64);
    if (k < h->M) k = h->M;
    if (k > 64) k = 64;
    CPB_TRY(adj.reserve(size_t(n) * h->M * 4 + 16));
    if (h->exact_edges) {
        // the legacy hybrid construction: exact nearest neighbours as candidates, links chosen on exact distances
        CPB_TRY(h->s_out.reserve(size_t(n) * k * 4 + 16));
        CPB_TRY(launch_exact_candidates(h, h->d_vectors.as<float>(), n, h->prune ? k : h->M, 0, n,
                                        h->prune ? h->s_out.as<uint32_t>() : adj.as<uint32_t>(), st));
        if (h->prune)
            CPB_TRY(launch_select_exact(h, h->d_vectors.as<float>(), n, h->s_out.as<uint32_t>(), k, 0, n, h->M, h->keep_pruned,
                                        adj.as<uint32_t>(), st));
        CPB_CUDA(cudaStreamSynchronize(st));
        return check_status(h);
    }
    if (!h->prune) {
        // build_with_gpu_knn(..., prune = false): the M nearest by (code distance, id) are the links
        CPB_TRY(launch_knn_graph(h, h->d_codes.p, n, h->M, 0, n, adj.as<uint32_t>(), nullptr, st));
        CPB_CUDA(cudaStreamSynchronize(st));
        return check_status(h);
    }
    CPB_TRY(h->s_out.reserve(size_t(n) * k * 4 + 16));
    CPB_TRY(launch_knn_graph(h, h->d_codes.p, n, k, 0, n, h->s_out.as<uint32_t>(), nullptr, st));
    if (h->rank_prune)
        CPB_TRY(launch_rank_prune(h, n, h->s_out.as<uint32_t>(), k, h->M, h->rank_pruning_alpha, adj.as<uint32_t>(), st));
    else
        CPB_TRY(launch_select_neighbors(h, h->d_codes.p, n, h->s_out.as<uint32_t>(), k, 0, n, h->M, h->keep_pruned,
                                        adj.as<uint32_t>(), st));
    CPB_CUDA(cudaStreamSynchronize(st));
    return check_status(h);
}

// A search call's lease on one of the handle's contexts: a free one of the right kind, a new one while
// the pool may grow, else the call waits for one to come back.
constexpr size_t kMaxWideCtx = 1;     // launches that fill the GPU gain nothing from running side by side
constexpr size_t kMaxNarrowCtx = 64;  // single-query calls from as many host threads
struct CtxLease {
    cphnsw_b200_index* h = nullptr;
    SearchCtx* cx = nullptr;
    int acquire(cphnsw_b200_index* h_, bool wide) {
        h = h_;
        std::unique_lock<std::mutex> lock(h->ctx_mu);
        for (;;) {
            size_t have = 0;
            for (auto& c : h->ctxs) {
                if (c->wide != wide) continue;
                ++have;
                if (!c->busy) {
                    c->busy = true;
                    cx = c.get();
                    return 0;
                }
            }
            if (have < (wide ? kMaxWideCtx : kMaxNarrowCtx)) {
                std::unique_ptr<SearchCtx> c(new SearchCtx());
                c->wide = wide;
                CPB_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
                CPB_CUDA(cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming));
                CPB_TRY(c->d_counter.reserve(16));
                c->busy = true;
                cx = c.get();
                h->ctxs.push_back(std::move(c));
                return 0;
            }
            h->ctx_cv.wait(lock);
        }
    }
    // work of this call goes to stream `st`: it must start behind whatever last used the scratch
    int begin(cudaStream_t st) {
        if (cx->pending) CPB_CUDA(cudaStreamWaitEvent(st, cx->done, 0));
        return 0;
    }
    // the call returns without having waited for `st`: the next user of the scratch has to
    int leave_pending(cudaStream_t st) {
        CPB_CUDA(cudaEventRecord(cx->done, st));
        cx->pending = true;
        return 0;
    }
    ~CtxLease() {
        if (!cx) return;
        {
            std::lock_guard<std::mutex> lock(h->ctx_mu);
            cx->busy = false;
        }
        h->ctx_cv.notify_one();
    }
};

// scan_only: brute_force_search (every node scored, no walk); calibrated: distances mapped through the fit;
// q_codes: the walk runs under the symmetric code distance to these query codes ([nq][K], same place as q).
// `st` is the caller's stream for device-pointer calls and nullptr for host-pointer calls, which run on the
// context's own stream and return with the results copied out.
int do_search(cphnsw_b200_index* h, const float* q, bool q_on_device, uint64_t nq, uint32_t k, uint32_t ef,
              uint32_t rerank_k, uint32_t* ids, float* dists, uint32_t* stats, bool out_on_device,
              cudaStream_t st, int scan_only = 0, bool calibrated = false, const void* q_codes = nullptr) {
    if (h->n == 0) {
        set_error("search on an empty index");
        return CPHNSW_B200_E_STATE;
    }
    if (k == 0 || (!q && !q_codes && nq) || !ids || !dists) {
        set_error("search: k must be > 0 and query/output pointers non-null");
        return CPHNSW_B200_E_INVALID;
    }
    uint32_t beam = ef > k ? ef : k;
    if (rerank_k > beam) beam = rerank_k;
    if (rerank_k && rerank_k < k) {
        set_error("search_and_rerank: rerank_k (%u) must be >= k (%u)", rerank_k, k);
        return CPHNSW_B200_E_INVALID;
    }
    if (beam > kMaxBeam) {
        set_error("search: beam width max(ef, k, rerank_k) must be <= %u (got %u)", kMaxBeam, beam);
        return CPHNSW_B200_E_INVALID;
    }
    if (nq == 0) return 0;
    CtxLease lease;
    CPB_TRY(lease.acquire(h, nq > kNarrowQueries));
    SearchCtx& cx = *lease.cx;
    const bool own_stream = !(q_on_device || out_on_device);
    if (own_stream) st = cx.stream;
    CPB_TRY(lease.begin(st));
    const uint64_t chunk = 16384;  // queries per launch: bounds the rotated-table scratch
    const size_t table_floats = size_t(h->K) * h->P;
    const size_t rb = code_row_bytes(h);
    bool synced = false;
    for (uint64_t q0 = 0; q0 < nq; q0 += chunk) {
        const uint64_t m = nq - q0 < chunk ? nq - q0 : chunk;
        synced = false;
        const float* dq = nullptr;
        const void* dqc = nullptr;  // query codes of a symmetric walk
        if (q_codes) {
            if (q_on_device) {
                dqc = static_cast<const unsigned char*>(q_codes) + q0 * rb;
            } else {
                CPB_TRY(cx.d_qcodes.reserve(m * rb + 16));
                CPB_CUDA(cudaMemcpyAsync(cx.d_qcodes.p, static_cast<const unsigned char*>(q_codes) + q0 * rb, m * rb,
                                         cudaMemcpyHostToDevice, st));
                dqc = cx.d_qcodes.p;
            }
        } else {
            if (q_on_device) {
                dq = q + q0 * h->dim;
            } else {
                CPB_TRY(cx.d_q.reserve(m * h->dim * 4));
                CPB_CUDA(cudaMemcpyAsync(cx.d_q.p, q + q0 * h->dim, m * h->dim * 4, cudaMemcpyHostToDevice, st));
                dq = cx.d_q.as<float>();
            }
            CPB_TRY(cx.d_qcodes.reserve(m * rb + 16));
            if (h->binary_codes) {
                // binary-code mode: the walk compares sign-bit codes (Hamming distance), no query table
                CPB_TRY(launch_encode(h, dq, m, cx.d_qcodes.p, nullptr, nullptr, st));
                dqc = cx.d_qcodes.p;
            } else {
                CPB_TRY(cx.d_qtables.reserve(m * table_floats * 4));
                CPB_TRY(launch_encode(h, dq, m, cx.d_qcodes.p, cx.d_qtables.as<float>(), nullptr, st));
            }
        }
        uint32_t *o_ids, *o_stats = nullptr;
        float* o_d;
        if (out_on_device) {
            o_ids = ids + q0 * k;
            o_d = dists + q0 * k;
            if (stats) o_stats = stats + q0 * 2;
        } else {
            CPB_TRY(cx.d_out_ids.reserve(m * k * 4));
            CPB_TRY(cx.d_out_dist.reserve(m * k * 4));
            o_ids = cx.d_out_ids.as<uint32_t>();
            o_d = cx.d_out_dist.as<float>();
            if (stats) {
                CPB_TRY(cx.d_stats.reserve(m * 8));
                o_stats = cx.d_stats.as<uint32_t>();
            }
        }
        CPB_TRY(launch_search(h, cx, dq, cx.d_qtables.as<float>(), m, k, beam, rerank_k, o_ids, o_d, o_stats, st, dqc,
                              scan_only));
        if (calibrated && rerank_k == 0) CPB_TRY(launch_affine(h, o_d, m * k, float(h->calib_alpha), float(h->calib_beta), st));
        if (!out_on_device) {
            CPB_CUDA(cudaMemcpyAsync(ids + q0 * k, o_ids, m * k * 4, cudaMemcpyDeviceToHost, st));
            CPB_CUDA(cudaMemcpyAsync(dists + q0 * k, o_d, m * k * 4, cudaMemcpyDeviceToHost, st));
            if (stats) CPB_CUDA(cudaMemcpyAsync(stats + q0 * 2, o_stats, m * 8, cudaMemcpyDeviceToHost, st));
            CPB_CUDA(cudaStreamSynchronize(st));
            synced = true;
        }
    }
    if (synced) cx.pending = false;
    else CPB_TRY(lease.leave_pending(st));
    return 0;
}

int do_calibrate(cphnsw_b200_index* h, uint64_t num_samples, uint64_t seed) {
    if (h->n == 0) {
        set_error("calibrate on an empty index");
        return CPHNSW_B200_E_STATE;
    }
    if (h->binary_codes) {
        set_error("calibrate: not available in binary-code mode (the distance is the Hamming distance itself)");
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    if (num_samples == 0 || num_samples > 65536) {
        set_error("calibrate: num_samples must be in 1..65536");
        return CPHNSW_B200_E_INVALID;
    }
    const uint32_t m = uint32_t(num_samples);
    std::vector<uint32_t> uv(size_t(m) * 2);
    std::mt19937_64 rng(seed);
    for (uint32_t s = 0; s < m; ++s) {
        uv[s] = uint32_t(rng() % h->n);
        uv[m + s] = uint32_t(rng() % h->n);
    }
    cudaStream_t st = 0;
    const size_t table_floats = size_t(h->K) * h->P;
    CPB_TRY(h->s_in.reserve(size_t(m) * 8 + 16));       // u, v
    CPB_TRY(h->s_out.reserve(size_t(m) * 8 + 16));      // x, y
    CPB_TRY(h->d_q.reserve(size_t(m) * h->dim * 4));    // the u vectors
    CPB_TRY(h->d_qtables.reserve(size_t(m) * table_floats * 4));
    CPB_TRY(h->d_qcodes.reserve(size_t(m) * code_row_bytes(h) + 16));
    uint32_t* d_u = h->s_in.as<uint32_t>();
    uint32_t* d_v = d_u + m;
    float* d_x = h->s_out.as<float>();
    float* d_y = d_x + m;
    CPB_CUDA(cudaMemcpyAsync(d_u, uv.data(), size_t(m) * 8, cudaMemcpyHostToDevice, st));
    CPB_TRY(gather_rows(h, h->d_vectors.p, h->dim * 4, d_u, m, h->d_q.p, st));
    CPB_TRY(launch_encode(h, h->d_q.as<float>(), m, h->d_qcodes.p, h->d_qtables.as<float>(), nullptr, st));
    CPB_TRY(launch_calibration_samples(h, h->d_qtables.as<float>(), d_u, d_v, m, d_x, d_y, st));
    std::vector<float> xy(size_t(m) * 2);
    CPB_CUDA(cudaMemcpyAsync(xy.data(), d_x, size_t(m) * 8, cudaMemcpyDeviceToHost, st));
    CPB_CUDA(cudaStreamSynchronize(st));
    // least squares in double on the host: 2 * num_samples floats
    const float* x = xy.data();
    const float* y = x + m;
    double sx = 0, sy = 0;
    for (uint32_t i = 0; i < m; ++i) sx += x[i], sy += y[i];
    const double mx = sx / m, my = sy / m;
    double sxx = 0, sxy = 0, syy = 0;
    for (uint32_t i = 0; i < m; ++i) {
        const double dx = x[i] - mx, dy = y[i] - my;
        sxx += dx * dx, sxy += dx * dy, syy += dy * dy;
    }
    h->calib_alpha = sxx > 0 ? sxy / sxx : 0.0;
    h->calib_beta = my - h->calib_alpha * mx;
    h->calib_r2 = (sxx > 0 && syy > 0) ? (sxy * sxy) / (sxx * syy) : 0.0;
    h->calib_samples = m;
    return 0;
}

// search_multiprobe: probe codes from the rotated queries, one symmetric-distance walk per probe,
// merge.  probe_codes_out (host, optional) receives the [nq][T][K] probe codes.
int do_multiprobe(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k, uint32_t ef, uint32_t T,
                  uint32_t* ids, float* dists, void* probe_codes_out, bool search) {
    if (T == 0 || T > 64) {
        set_error("search_multiprobe: num_probes must be in 1..64 (got %u)", T);
        return CPHNSW_B200_E_INVALID;
    }
    if (h->binary_codes) {
        set_error("search_multiprobe: not available in binary-code mode");
        return CPHNSW_B200_E_UNSUPPORTED;
    }
    if (!q && nq) {
        set_error("search_multiprobe: null query pointer");
        return CPHNSW_B200_E_INVALID;
    }
    uint32_t beam = ef > k ? ef : k;
    if (search) {
        if (h->n == 0) {
            set_error("search on an empty index");
            return CPHNSW_B200_E_STATE;
        }
        if (k == 0 || !ids || !dists) {
            set_error("search_multiprobe: k must be > 0 and output pointers non-null");
            return CPHNSW_B200_E_INVALID;
        }
        if (beam > 1024 || uint64_t(T) * k > 2048) {
            set_error("search_multiprobe: need max(ef,k) <= 1024 and num_probes*k <= 2048");
            return CPHNSW_B200_E_INVALID;
        }
    }
    if (nq == 0) return 0;
    const uint64_t chunk = 4096;
    const size_t table_floats = size_t(h->K) * h->P;
    const size_t rb = code_row_bytes(h);
    CtxLease lease;
    CPB_TRY(lease.acquire(h, (nq < chunk ? nq : chunk) * T > kNarrowQueries));
    SearchCtx& cx = *lease.cx;
    cudaStream_t st = cx.stream;
    CPB_TRY(lease.begin(st));
    for (uint64_t q0 = 0; q0 < nq; q0 += chunk) {
        const uint64_t m = nq - q0 < chunk ? nq - q0 : chunk;
        CPB_TRY(cx.d_q.reserve(m * h->dim * 4));
        CPB_CUDA(cudaMemcpyAsync(cx.d_q.p, q + q0 * h->dim, m * h->dim * 4, cudaMemcpyHostToDevice, st));
        CPB_TRY(cx.d_qtables.reserve(m * table_floats * 4));
        CPB_TRY(cx.d_qcodes.reserve(m * rb + 16));
        CPB_TRY(launch_encode(h, cx.d_q.as<float>(), m, cx.d_qcodes.p, cx.d_qtables.as<float>(), nullptr, st));
        CPB_TRY(cx.d_probe_codes.reserve(m * T * rb + 16));
        CPB_TRY(launch_probe_codes(h, cx.d_qtables.as<float>(), m, T, cx.d_probe_codes.p, st));
        if (probe_codes_out)
            CPB_CUDA(cudaMemcpyAsync((char*)probe_codes_out + q0 * T * rb, cx.d_probe_codes.p, m * T * rb,
                                     cudaMemcpyDeviceToHost, st));
        if (search) {
            CPB_TRY(cx.d_probe_ids.reserve(m * T * k * 4));
            CPB_TRY(cx.d_probe_dist.reserve(m * T * k * 4));
            CPB_TRY(cx.d_out_ids.reserve(m * k * 4));
            CPB_TRY(cx.d_out_dist.reserve(m * k * 4));
            CPB_TRY(launch_search(h, cx, nullptr, nullptr, m * T, k, beam, 0, cx.d_probe_ids.as<uint32_t>(),
                                  cx.d_probe_dist.as<float>(), nullptr, st, cx.d_probe_codes.p));
            CPB_TRY(launch_merge_probes(h, cx.d_probe_ids.as<uint32_t>(), cx.d_probe_dist.as<float>(), m, T, k,
                                        cx.d_out_ids.as<uint32_t>(), cx.d_out_dist.as<float>(), st));
            CPB_CUDA(cudaMemcpyAsync(ids + q0 * k, cx.d_out_ids.p, m * k * 4, cudaMemcpyDeviceToHost, st));
            CPB_CUDA(cudaMemcpyAsync(dists + q0 * k, cx.d_out_dist.p, m * k * 4, cudaMemcpyDeviceToHost, st));
        }
        CPB_CUDA(cudaStreamSynchronize(st));
    }
    cx.pending = false;
    return 0;
}

}  // namespace
}  // namespace cpb

using namespace cpb;

cphnsw_b200_index::~cphnsw_b200_index() {
    for (auto& pool : events)
        for (auto& e : pool) {
            if (e.start) cudaEventDestroy(e.start);
            if (e.stop) cudaEventDestroy(e.stop);
        }
}

extern "C" {

int cphnsw_b200_kernel_time(cphnsw_b200_index* h, int kind, double* total_ms, uint64_t* launches) {
    CPB_TRY(bind(h));
    if (kind < 0 || kind >= kKernelKinds || !total_ms || !launches) {
        set_error("kernel_time: bad argument");
        return CPHNSW_B200_E_INVALID;
    }
    std::lock_guard<std::mutex> lock(h->ev_mu);
    double sum = 0.0;
    for (size_t i = 0; i < h->events_used[kind]; ++i) {
        float ms = 0.f;
        CPB_CUDA(cudaEventSynchronize(h->events[kind][i].stop));
        CPB_CUDA(cudaEventElapsedTime(&ms, h->events[kind][i].start, h->events[kind][i].stop));
        sum += ms;
    }
    *total_ms = sum;
    *launches = h->events_used[kind];
    h->events_used[kind] = 0;
    return 0;
}

const char* cphnsw_b200_last_error(void) { return g_error.c_str(); }

int cphnsw_b200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int ok = 0;
    for (int d = 0; d < n; ++d) {
        cudaDeviceProp p;
        if (cudaGetDeviceProperties(&p, d) == cudaSuccess && p.major == 10) ++ok;
    }
    return ok;
}

static int create_impl(uint64_t dim, uint32_t K, uint32_t component_bytes, uint32_t M, uint32_t ef_construction,
                       uint64_t seed, int fht_convention, int device, bool binary, cphnsw_b200_index** out) {
    if (!out) {
        set_error("create: out is null");
        return CPHNSW_B200_E_INVALID;
    }
    *out = nullptr;
    // bounds of CPHNSWParams::finalize (include/cphnsw/core/types.hpp:403-469)
    if (dim == 0) { set_error("CPHNSWParams: dim must be > 0"); return CPHNSW_B200_E_INVALID; }
    if (K == 0) { set_error("CPHNSWParams: k (code width) must be > 0"); return CPHNSW_B200_E_INVALID; }
    if (K > 256) { set_error("CPHNSWParams: k (code width) must be <= 256"); return CPHNSW_B200_E_INVALID; }
    if (M == 0) { set_error("CPHNSWParams: M (max connections) must be > 0"); return CPHNSW_B200_E_INVALID; }
    if (M > 64) { set_error("CPHNSWParams: M must be <= 64 (FLASH_MAX_M limit)"); return CPHNSW_B200_E_INVALID; }
    if (ef_construction < M) {
        set_error("CPHNSWParams: ef_construction must be >= M for good graph quality");
        return CPHNSW_B200_E_INVALID;
    }
    if (ef_construction > 10000) { set_error("CPHNSWParams: ef_construction must be <= 10000"); return CPHNSW_B200_E_INVALID; }
    if (component_bytes != 1 && component_bytes != 2) {
        set_error("component_bytes must be 1 (uint8_t) or 2 (uint16_t)");
        return CPHNSW_B200_E_INVALID;
    }
    if (fht_convention < 0 || fht_convention > 2) { set_error("unknown fht_convention %d", fht_convention); return CPHNSW_B200_E_INVALID; }
    // the encode kernels serve padded dims up to 32768 (a uint16 component holds no more), 65536 for sign-bit codes
    if (dim > (binary ? 65536u : 32768u)) {
        set_error("dim %llu is too large (max %u)", (unsigned long long)dim, binary ? 65536u : 32768u);
        return CPHNSW_B200_E_INVALID;
    }
    const uint64_t P = next_pow2(dim);
    // a component holds (index << 1) | sign (types.hpp:88-90)
    if (!binary && ((component_bytes == 1 && P > 128) || (component_bytes == 2 && P > 32768))) {
        set_error("padded dim %llu does not fit a %u-byte component (max %d)", (unsigned long long)P,
                  component_bytes, component_bytes == 1 ? 128 : 32768);
        return CPHNSW_B200_E_INVALID;
    }
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        set_error("no CUDA device available: this library has no CPU path");
        return CPHNSW_B200_E_CUDA;
    }
    if (device < 0 || device >= ndev) { set_error("device %d out of range (%d devices)", device, ndev); return CPHNSW_B200_E_INVALID; }
    cudaDeviceProp prop;
    CPB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
        return CPHNSW_B200_E_CUDA;
    }
    CPB_CUDA(cudaSetDevice(device));
    cphnsw_b200_index* h = nullptr;
    try {
        h = new cphnsw_b200_index();
        h->signs.resize(size_t(K) * 3 * P);
    } catch (const std::exception&) {  // nothing may leave an extern "C" entry point as an exception
        delete h;
        set_error("create: out of host memory");
        return CPHNSW_B200_E_INVALID;
    }
    h->dim = dim;
    h->P = P;
    h->K = K;
    h->comp_bytes = component_bytes;
    h->M = M;
    h->ef_construction = ef_construction;
    h->seed = seed;
    h->convention = fht_convention;
    h->device = device;
    h->binary_codes = binary ? 1 : 0;
    h->sm_count = prop.multiProcessorCount;
    // RotationChain: rotation r is seeded seed + r (include/cphnsw/encoder/rotation.hpp:173-178);
    // each table is drawn layer by layer from mt19937_64 through uniform_int_distribution<int>(0,1)
    // (rotation.hpp:134-144) — the standard library does the draw, as in the reference.
    for (uint32_t r = 0; r < K; ++r) {
        std::mt19937_64 rng(seed + r);
        std::uniform_int_distribution<int> coin(0, 1);
        for (int l = 0; l < 3; ++l)
            for (uint64_t i = 0; i < P; ++i) h->signs[(size_t(r) * 3 + l) * P + i] = coin(rng) ? 1 : -1;
    }
    int rc = upload_signs(h);
    h->events[0].reserve(1024);  // LaunchTimer keeps pointers into these pools
    for (int kk = 1; kk < kKernelKinds; ++kk) h->events[kk].reserve(1024);
    if (rc == 0) rc = h->d_status.reserve(256);
    if (rc == 0 && cudaMemset(h->d_status.p, 0, 256) != cudaSuccess) rc = cuda_fail(cudaGetLastError(), "memset status");
    if (rc != 0) {
        delete h;
        return rc;
    }
    *out = h;
    return 0;
}

int cphnsw_b200_create(uint64_t dim, uint32_t K, uint32_t component_bytes, uint32_t M, uint32_t ef_construction,
                       uint64_t seed, int fht_convention, int device, cphnsw_b200_index** out) {
    return create_impl(dim, K, component_bytes, M, ef_construction, seed, fht_convention, device, false, out);
}

// binary-code mode from the start: a component holds a sign bit only, so one byte does for every dimension
int cphnsw_b200_create_binary(uint64_t dim, uint32_t K, uint32_t M, uint32_t ef_construction, uint64_t seed,
                              int fht_convention, int device, cphnsw_b200_index** out) {
    return create_impl(dim, K, 1, M, ef_construction, seed, fht_convention, device, true, out);
}

int cphnsw_b200_destroy(cphnsw_b200_index* h) {
    if (!h) return 0;
    cudaSetDevice(h->device);
    delete h;
    return 0;
}

int cphnsw_b200_set_param(cphnsw_b200_index* h, const char* name, double v) {
    if (!h || !name) { set_error("set_param: null argument"); return CPHNSW_B200_E_INVALID; }
    std::string s(name);
    if (s == "keep_pruned") { h->keep_pruned = v != 0.0; return 0; }
    if (s == "prune") { h->prune = v != 0.0; return 0; }
    if (s == "profile") { h->profile = v != 0.0; return 0; }
    if (s == "knn_kernel") {
        if (v != 0 && v != 1 && v != 2) { set_error("knn_kernel must be 0 (pick), 1 (byte-wise) or 2 (bit-sliced)"); return CPHNSW_B200_E_INVALID; }
        h->knn_kernel = int(v);
        return 0;
    }
    if (s == "search_kernel") {
        if (v != 0 && v != 1 && v != 2) { set_error("search_kernel must be 0 (pick), 1 (one warp per query) or 2 (two warps per query)"); return CPHNSW_B200_E_INVALID; }
        h->search_kernel = int(v);
        return 0;
    }
    if (s == "search_table_smem") { h->search_table_smem = v != 0.0; return 0; }
    if (s == "binary_codes") {
        if (v != 0 && v != 1) { set_error("binary_codes must be 0 or 1"); return CPHNSW_B200_E_INVALID; }
        if (h->n && int(v) != h->binary_codes) { set_error("binary_codes cannot change once vectors have been added"); return CPHNSW_B200_E_STATE; }
        if (v == 0 && h->residual_bits) { set_error("binary_codes cannot be switched off while residual_bits is set"); return CPHNSW_B200_E_INVALID; }
        // a full component holds (index << 1) | sign: the bound create checks for the K-byte codes
        if (v == 0 && ((h->comp_bytes == 1 && h->P > 128) || (h->comp_bytes == 2 && h->P > 32768))) {
            set_error("binary_codes cannot be switched off: padded dim %llu does not fit a %u-byte component", (unsigned long long)h->P, h->comp_bytes);
            return CPHNSW_B200_E_INVALID;
        }
        h->binary_codes = int(v);
        return 0;
    }
    if (s == "residual_bits" || s == "residual_shift") {
        // residual codes of the unified index (ResidualCode<K, R>, include/cphnsw/core/codes.hpp:76-129;
        // combined distance include/cphnsw/core/types.hpp:284-302)
        if (h->n) { set_error("%s cannot change once vectors have been added", name); return CPHNSW_B200_E_STATE; }
        if (s == "residual_shift") {
            if (v < 0 || v > 4 || v != double(int(v))) { set_error("residual_shift must be in 0..4"); return CPHNSW_B200_E_INVALID; }
            h->residual_shift = uint32_t(v);
            return 0;
        }
        if (v != 0 && !h->binary_codes) { set_error("residual_bits needs binary_codes = 1"); return CPHNSW_B200_E_INVALID; }
        if (v < 0 || v >= h->K || v != double(int(v))) { set_error("residual_bits must be in 0..K-1 (K = primary + residual bits = %u)", h->K); return CPHNSW_B200_E_INVALID; }
        if (v != 0 && ((h->K - uint32_t(v)) * h->comp_bytes) % 4 != 0) {
            set_error("residual_bits: the primary part (K - residual_bits components) must fill whole 32-bit words");
            return CPHNSW_B200_E_INVALID;
        }
        h->residual_bits = uint32_t(v);
        return 0;
    }
    if (s == "first_wait_polls") {
        if (v < 0 || v > 4194304.0) { set_error("first_wait_polls must be in 0..2^22"); return CPHNSW_B200_E_INVALID; }
        h->first_wait_polls = uint32_t(v);
        return 0;
    }
    if (s == "rank_prune") { h->rank_prune = v != 0.0; return 0; }
    if (s == "exact_edges") { h->exact_edges = v != 0.0; return 0; }
    if (s == "rank_pruning_alpha") {
        // bounds of CPHNSWParams::finalize (include/cphnsw/core/types.hpp:459-466)
        if (!(v >= 1.0)) { set_error("CPHNSWParams: rank_pruning_alpha must be >= 1.0"); return CPHNSW_B200_E_INVALID; }
        if (v > 3.0) { set_error("CPHNSWParams: rank_pruning_alpha must be <= 3.0"); return CPHNSW_B200_E_INVALID; }
        h->rank_pruning_alpha = float(v);
        return 0;
    }
    if (s == "build_seed") {
        if (v < 0 || v > 2147483647.0) { set_error("build_seed must be in 0..2^31-1 (0 = exact kNN graph over everything)"); return CPHNSW_B200_E_INVALID; }
        h->build_seed = uint32_t(v);
        return 0;
    }
    if (s == "k_entry") {
        if (v < 1) { set_error("CPHNSWParams: k_entry must be > 0"); return CPHNSW_B200_E_INVALID; }
        if (v > 100) { set_error("CPHNSWParams: k_entry must be <= 100"); return CPHNSW_B200_E_INVALID; }
        h->k_entry = uint32_t(v);
    } else if (s == "knn_k") {
        if (v < 0 || v > 64) { set_error("knn_k must be in 0..64 (0 = default)"); return CPHNSW_B200_E_INVALID; }
        h->knn_k = uint32_t(v);
        return 0;
    } else if (s == "entry_scan") {
        if (v < 0 || v > 1048576) { set_error("entry_scan must be in 0..1048576 (0 = k_entry)"); return CPHNSW_B200_E_INVALID; }
        h->entry_scan = uint32_t(v);
    } else {
        set_error("unknown parameter '%s'", name);
        return CPHNSW_B200_E_INVALID;
    }
    if (h->n) {
        CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
        return set_entry_ids(h);
    }
    return 0;
}

int cphnsw_b200_get_param(const cphnsw_b200_index* h, const char* name, double* v) {
    if (!h || !name || !v) { set_error("get_param: null argument"); return CPHNSW_B200_E_INVALID; }
    std::string s(name);
    if (s == "keep_pruned") *v = h->keep_pruned;
    else if (s == "prune") *v = h->prune;
    else if (s == "profile") *v = h->profile;
    else if (s == "knn_kernel") *v = h->knn_kernel;
    else if (s == "search_kernel") *v = h->search_kernel;
    else if (s == "search_table_smem") *v = h->search_table_smem;
    else if (s == "build_seed") *v = h->build_seed;
    else if (s == "first_wait_polls") *v = h->first_wait_polls;
    else if (s == "rank_prune") *v = h->rank_prune;
    else if (s == "exact_edges") *v = h->exact_edges;
    else if (s == "rank_pruning_alpha") *v = h->rank_pruning_alpha;
    else if (s == "binary_codes") *v = h->binary_codes;
    else if (s == "stored_code_bytes")  // bytes of HBM a node's code takes while no build stage runs
        *v = h->codes_released ? double(h->packed_words) * 4.0 : double(h->K) * h->comp_bytes;
    else if (s == "residual_bits") *v = h->residual_bits;
    else if (s == "residual_shift") *v = h->residual_shift;
    else if (s == "k_entry") *v = h->k_entry;
    else if (s == "knn_k") *v = h->knn_k;
    else if (s == "entry_scan") *v = h->entry_scan;
    else if (s == "M") *v = h->M;
    else if (s == "K") *v = h->K;
    else if (s == "ef_construction") *v = h->ef_construction;
    else if (s == "component_bytes") *v = h->comp_bytes;
    else { set_error("unknown parameter '%s'", name); return CPHNSW_B200_E_INVALID; }
    return 0;
}

uint64_t cphnsw_b200_dim(const cphnsw_b200_index* h) { return h ? h->dim : 0; }
uint64_t cphnsw_b200_padded_dim(const cphnsw_b200_index* h) { return h ? h->P : 0; }
uint64_t cphnsw_b200_size(const cphnsw_b200_index* h) { return h ? h->n : 0; }
uint64_t cphnsw_b200_launch_count(const cphnsw_b200_index* h) { return h ? h->launches.load() : uint64_t(0); }

int cphnsw_b200_get_sign_tables(const cphnsw_b200_index* h, int8_t* out) {
    if (!h || !out) { set_error("get_sign_tables: null argument"); return CPHNSW_B200_E_INVALID; }
    std::memcpy(out, h->signs.data(), h->signs.size());
    return 0;
}

int cphnsw_b200_set_sign_tables(cphnsw_b200_index* h, const int8_t* signs) {
    if (!h || !signs) { set_error("set_sign_tables: null argument"); return CPHNSW_B200_E_INVALID; }
    for (size_t i = 0; i < h->signs.size(); ++i)
        if (signs[i] != 1 && signs[i] != -1) { set_error("sign tables must hold +1/-1 only"); return CPHNSW_B200_E_INVALID; }
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    std::memcpy(h->signs.data(), signs, h->signs.size());
    return upload_signs(h);
}

int cphnsw_b200_check_device_status(cphnsw_b200_index* h) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    return check_status(h);
}

// ---- device-pointer entry points ---------------------------------------------------------------------
int cphnsw_b200_encode_dev(cphnsw_b200_index* h, const float* d_x, uint64_t n, void* d_codes, float* d_rotated,
                           float* d_magnitudes, void* stream) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (n && (!d_x || !d_codes)) { set_error("encode: null pointer"); return CPHNSW_B200_E_INVALID; }
    return launch_encode(h, d_x, n, d_codes, d_rotated, d_magnitudes, (cudaStream_t)stream);
}

int cphnsw_b200_code_distance_dev(cphnsw_b200_index* h, const void* d_a, uint64_t na, const void* d_b, uint64_t nb,
                                  uint16_t* d_out, void* stream) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (na && nb && (!d_a || !d_b || !d_out)) { set_error("code_distance: null pointer"); return CPHNSW_B200_E_INVALID; }
    return launch_code_distance(h, d_a, na, d_b, nb, d_out, (cudaStream_t)stream);
}

int cphnsw_b200_knn_graph_dev(cphnsw_b200_index* h, const void* d_codes, uint64_t n, uint32_t k, uint64_t row_begin,
                              uint64_t row_end, uint32_t* d_nbrs, uint16_t* d_dist, void* stream) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (row_end > row_begin && (!d_codes || !d_nbrs)) { set_error("knn_graph: null pointer"); return CPHNSW_B200_E_INVALID; }
    return launch_knn_graph(h, d_codes, n, k, row_begin, row_end, d_nbrs, d_dist, (cudaStream_t)stream);
}

int cphnsw_b200_select_neighbors_dev(cphnsw_b200_index* h, const void* d_codes, uint64_t n, const uint32_t* d_cand,
                                     uint32_t k, uint64_t row_begin, uint64_t row_end, uint32_t M, int keep_pruned,
                                     uint32_t* d_adj, void* stream) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (row_end > row_begin && (!d_codes || !d_cand || !d_adj)) { set_error("select_neighbors: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (row_end > n) { set_error("select_neighbors: row range exceeds n"); return CPHNSW_B200_E_INVALID; }
    return launch_select_neighbors(h, d_codes, n, d_cand, k, row_begin, row_end, M, keep_pruned, d_adj,
                                   (cudaStream_t)stream);
}

int cphnsw_b200_install_dev(cphnsw_b200_index* h, const float* d_vectors, const void* d_codes, const uint32_t* d_adj,
                            uint64_t n, void* stream) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (n == 0 || !d_vectors || !d_codes || !d_adj) { set_error("install: null pointer or n == 0"); return CPHNSW_B200_E_INVALID; }
    if (n >= 0x80000000ull) { set_error("install: n must be < 2^31 (the top bit of a node id is used by the search)"); return CPHNSW_B200_E_INVALID; }
    cudaStream_t st = (cudaStream_t)stream;
    CPB_TRY(h->d_vectors.reserve(n * h->dim * 4));
    CPB_TRY(h->d_codes.reserve(n * code_row_bytes(h) + 16));
    h->codes_released = false;  // the codes are replaced as a whole
    CPB_TRY(h->d_adj.reserve(n * h->M * 4 + 16));
    CPB_CUDA(cudaMemcpyAsync(h->d_vectors.p, d_vectors, n * h->dim * 4, cudaMemcpyDeviceToDevice, st));
    CPB_CUDA(cudaMemcpyAsync(h->d_codes.p, d_codes, n * code_row_bytes(h), cudaMemcpyDeviceToDevice, st));
    CPB_CUDA(cudaMemcpyAsync(h->d_adj.p, d_adj, n * h->M * 4, cudaMemcpyDeviceToDevice, st));
    CPB_CUDA(cudaStreamSynchronize(st));
    h->n = n;
    drop_search_scratch(h);
    return set_entry_ids(h);
}

int cphnsw_b200_install(cphnsw_b200_index* h, const float* vectors, const void* codes, const uint32_t* adj, uint64_t n) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (n == 0 || !vectors || !codes || !adj) { set_error("install: null pointer or n == 0"); return CPHNSW_B200_E_INVALID; }
    if (n >= 0x80000000ull) { set_error("install: n must be < 2^31 (the top bit of a node id is used by the search)"); return CPHNSW_B200_E_INVALID; }
    const size_t rb = code_row_bytes(h);
    CPB_TRY(h->d_vectors.reserve(n * h->dim * 4));
    CPB_TRY(h->d_codes.reserve(n * rb + 16));
    h->codes_released = false;  // the codes are replaced as a whole
    CPB_TRY(h->d_adj.reserve(n * h->M * 4 + 16));
    CPB_CUDA(cudaMemcpy(h->d_vectors.p, vectors, n * h->dim * 4, cudaMemcpyHostToDevice));
    CPB_CUDA(cudaMemcpy(h->d_codes.p, codes, n * rb, cudaMemcpyHostToDevice));
    CPB_CUDA(cudaMemcpy(h->d_adj.p, adj, n * h->M * 4, cudaMemcpyHostToDevice));
    h->n = n;
    drop_search_scratch(h);
    return set_entry_ids(h);
}

int cphnsw_b200_search_codes_batch(cphnsw_b200_index* h, const void* qcodes, uint64_t nq, uint32_t k, uint32_t ef,
                                   uint32_t* ids_out, float* dists_out, uint32_t* stats_out) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    return do_search(h, nullptr, false, nq, k, ef, 0, ids_out, dists_out, stats_out, false, nullptr, 0, false, qcodes);
}

int cphnsw_b200_get_code(const cphnsw_b200_index* h, uint32_t id, void* code_out) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    if (!code_out) { set_error("get_code: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (id >= h->n) { set_error("get_code: node %u does not exist (size %llu)", id, (unsigned long long)h->n); return CPHNSW_B200_E_INVALID; }
    const size_t rb = code_row_bytes(h);
    if (h->codes_released) return host_codes_from_packed(h, id, 1, static_cast<unsigned char*>(code_out));
    CPB_CUDA(cudaMemcpy(code_out, h->d_codes.as<unsigned char>() + size_t(id) * rb, rb, cudaMemcpyDeviceToHost));
    return 0;
}

int cphnsw_b200_search_dev(cphnsw_b200_index* h, const float* d_q, uint64_t nq, uint32_t k, uint32_t ef,
                           uint32_t rerank_k, uint32_t* d_ids, float* d_dists, uint32_t* d_stats, void* stream) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    return do_search(h, d_q, true, nq, k, ef, rerank_k, d_ids, d_dists, d_stats, true, (cudaStream_t)stream);
}

int cphnsw_b200_brute_force_search_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k, uint32_t* ids_out,
                                         float* dists_out) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    return do_search(h, q, false, nq, k, k, 0, ids_out, dists_out, nullptr, false, 0, 1);
}

// the vectors exact_search / rerank run over: those of set_exact_base if any, else the index's own
static const float* exact_vectors(cphnsw_b200_index* h, uint64_t* n) {
    if (h->n_exact) {
        *n = h->n_exact;
        return h->d_exact_base.as<float>();
    }
    *n = h->n;
    return h->d_vectors.as<float>();
}

int cphnsw_b200_set_exact_base(cphnsw_b200_index* h, const float* base, uint64_t n) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (n == 0) {
        h->d_exact_base.release();
        h->n_exact = 0;
        return 0;
    }
    if (!base) { set_error("set_exact_base: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (n >= kInvalidNode) { set_error("set_exact_base: at most 2^32 - 2 vectors"); return CPHNSW_B200_E_INVALID; }
    h->n_exact = 0;
    CPB_TRY(h->d_exact_base.reserve(n * h->dim * sizeof(float)));
    CPB_CUDA(cudaMemcpy(h->d_exact_base.p, base, n * h->dim * sizeof(float), cudaMemcpyHostToDevice));
    h->n_exact = n;
    return 0;
}

int cphnsw_b200_exact_search_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k, uint32_t* ids_out,
                                   float* dists_out) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (nq == 0) return 0;
    if (!q || !ids_out || !dists_out) { set_error("exact_search: null pointer"); return CPHNSW_B200_E_INVALID; }
    uint64_t n = 0;
    const float* base = exact_vectors(h, &n);
    if (n == 0) { set_error("exact_search: no vectors (empty index and no exact base)"); return CPHNSW_B200_E_STATE; }
    CPB_TRY(h->s_in.reserve(nq * h->dim * sizeof(float)));
    CPB_TRY(h->s_out.reserve(nq * k * 4 + 16));
    CPB_TRY(h->s_out2.reserve(nq * k * 4 + 16));
    CPB_CUDA(cudaMemcpy(h->s_in.p, q, nq * h->dim * sizeof(float), cudaMemcpyHostToDevice));
    CPB_TRY(launch_exact_search(h, base, n, h->s_in.as<float>(), nq, k, h->s_out.as<uint32_t>(), h->s_out2.as<float>(), 0));
    CPB_CUDA(cudaMemcpy(ids_out, h->s_out.p, nq * k * 4, cudaMemcpyDeviceToHost));
    CPB_CUDA(cudaMemcpy(dists_out, h->s_out2.p, nq * k * 4, cudaMemcpyDeviceToHost));
    return 0;
}

int cphnsw_b200_exact_search_dev(cphnsw_b200_index* h, const float* d_base, uint64_t n, const float* d_q, uint64_t nq,
                                 uint32_t k, uint32_t* d_ids, float* d_dists, void* stream) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (nq == 0) return 0;
    if ((n && !d_base) || !d_q || !d_ids || !d_dists) { set_error("exact_search: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (n >= kInvalidNode) { set_error("exact_search: at most 2^32 - 2 vectors"); return CPHNSW_B200_E_INVALID; }
    return launch_exact_search(h, d_base, n, d_q, nq, k, d_ids, d_dists, (cudaStream_t)stream);
}

int cphnsw_b200_rerank_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, const uint32_t* cand, uint32_t num_cand,
                             uint32_t k, uint32_t* ids_out, float* dists_out) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (nq == 0) return 0;
    if (!q || (num_cand && !cand) || !ids_out || !dists_out) { set_error("rerank: null pointer"); return CPHNSW_B200_E_INVALID; }
    uint64_t n = 0;
    const float* base = exact_vectors(h, &n);
    if (n == 0) { set_error("rerank: no vectors (empty index and no exact base)"); return CPHNSW_B200_E_STATE; }
    CPB_TRY(h->s_in.reserve(nq * h->dim * sizeof(float)));
    CPB_TRY(h->s_in2.reserve(nq * uint64_t(num_cand) * 4 + 16));
    CPB_TRY(h->s_out.reserve(nq * k * 4 + 16));
    CPB_TRY(h->s_out2.reserve(nq * k * 4 + 16));
    CPB_CUDA(cudaMemcpy(h->s_in.p, q, nq * h->dim * sizeof(float), cudaMemcpyHostToDevice));
    if (num_cand) CPB_CUDA(cudaMemcpy(h->s_in2.p, cand, nq * uint64_t(num_cand) * 4, cudaMemcpyHostToDevice));
    CPB_TRY(launch_rerank(h, base, n, h->s_in.as<float>(), nq, h->s_in2.as<uint32_t>(), num_cand, k, h->s_out.as<uint32_t>(),
                          h->s_out2.as<float>(), 0));
    CPB_CUDA(cudaMemcpy(ids_out, h->s_out.p, nq * k * 4, cudaMemcpyDeviceToHost));
    CPB_CUDA(cudaMemcpy(dists_out, h->s_out2.p, nq * k * 4, cudaMemcpyDeviceToHost));
    return 0;
}

int cphnsw_b200_verify_connectivity(cphnsw_b200_index* h, uint64_t* reachable_out) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (!reachable_out) { set_error("verify_connectivity: null pointer"); return CPHNSW_B200_E_INVALID; }
    *reachable_out = 0;
    if (h->n == 0) return 0;
    return launch_connectivity(h, reachable_out, 0);
}

int cphnsw_b200_calibrate(cphnsw_b200_index* h, uint64_t num_samples, uint64_t seed, double* alpha_out, double* beta_out,
                          double* r_squared_out) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    CPB_TRY(do_calibrate(h, num_samples, seed));
    if (alpha_out) *alpha_out = h->calib_alpha;
    if (beta_out) *beta_out = h->calib_beta;
    if (r_squared_out) *r_squared_out = h->calib_r2;
    return 0;
}

int cphnsw_b200_get_calibration(const cphnsw_b200_index* h, double* alpha_out, double* beta_out, double* r_squared_out,
                                uint64_t* num_samples_out) {
    if (!h) { set_error("null index handle"); return CPHNSW_B200_E_INVALID; }
    if (alpha_out) *alpha_out = h->calib_alpha;
    if (beta_out) *beta_out = h->calib_beta;
    if (r_squared_out) *r_squared_out = h->calib_r2;
    if (num_samples_out) *num_samples_out = h->calib_samples;
    return 0;
}

int cphnsw_b200_search_calibrated_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k, uint32_t ef,
                                        uint32_t rerank_k, uint32_t* ids_out, float* dists_out) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    return do_search(h, q, false, nq, k, ef, rerank_k, ids_out, dists_out, nullptr, false, 0, 0, true);
}

int cphnsw_b200_get_binary_codes(const cphnsw_b200_index* h, uint64_t* words_out) {
    if (!h || (!words_out && h->n)) { set_error("get_binary_codes: null argument"); return CPHNSW_B200_E_INVALID; }
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (h->n == 0) return 0;
    cphnsw_b200_index* m = const_cast<cphnsw_b200_index*>(h);  // scratch and launch counter only
    const size_t bytes = h->n * ((h->K + 63) / 64) * 8;
    if (h->codes_released) {
        // the stored code is the packed bits already, 32 per word: two words make one of the output's
        const size_t pw = size_t(h->packed_words), nw = (h->K + 63) / 64;
        std::vector<uint32_t> w(h->n * pw);
        CPB_CUDA(cudaMemcpy(w.data(), h->d_packed.p, w.size() * 4, cudaMemcpyDeviceToHost));
        for (uint64_t i = 0; i < h->n; ++i)
            for (size_t j = 0; j < nw; ++j) {
                const uint64_t lo = w[i * pw + 2 * j];
                const uint64_t hi = 2 * j + 1 < pw ? w[i * pw + 2 * j + 1] : 0;
                words_out[i * nw + j] = lo | (hi << 32);
            }
        return 0;
    }
    CPB_TRY(m->s_out.reserve(bytes));
    CPB_TRY(launch_pack_sign_bits(m, h->d_codes.p, h->n, m->s_out.as<uint64_t>(), 0));
    CPB_CUDA(cudaMemcpy(words_out, m->s_out.p, bytes, cudaMemcpyDeviceToHost));
    return 0;
}

// ---- index file -------------------------------------------------------------------------------------------
namespace {
constexpr char kFileMagic[8] = {'C', 'P', 'H', 'N', 'S', 'W', 'B', '2'};
constexpr uint32_t kFileVersion = 1;
struct FileHeader {  // after the magic; all little-endian, naturally aligned
    uint32_t version, K, comp_bytes, M, ef_construction, keep_pruned, k_entry, knn_k, entry_scan;
    int32_t convention;
    uint32_t binary_codes, residual;  // residual = residual_bits | residual_shift << 16
    uint64_t dim, seed, n, calib_samples;
    double calib_alpha, calib_beta, calib_r2;
};
struct FileCloser {
    std::FILE* f;
    ~FileCloser() { if (f) std::fclose(f); }
};
// device -> file in pieces through a host buffer
int write_device(std::FILE* f, const void* d, size_t bytes, std::vector<char>& buf) {
    for (size_t off = 0; off < bytes; off += buf.size()) {
        const size_t m = bytes - off < buf.size() ? bytes - off : buf.size();
        CPB_CUDA(cudaMemcpy(buf.data(), static_cast<const char*>(d) + off, m, cudaMemcpyDeviceToHost));
        if (std::fwrite(buf.data(), 1, m, f) != m) { set_error("save: write failed"); return CPHNSW_B200_E_INVALID; }
    }
    return 0;
}
int read_device(std::FILE* f, void* d, size_t bytes, std::vector<char>& buf) {
    for (size_t off = 0; off < bytes; off += buf.size()) {
        const size_t m = bytes - off < buf.size() ? bytes - off : buf.size();
        if (std::fread(buf.data(), 1, m, f) != m) { set_error("load: file is shorter than its header says"); return CPHNSW_B200_E_INVALID; }
        CPB_CUDA(cudaMemcpy(static_cast<char*>(d) + off, buf.data(), m, cudaMemcpyHostToDevice));
    }
    return 0;
}
}  // namespace

int cphnsw_b200_save(cphnsw_b200_index* h, const char* path) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (!path) { set_error("save: null path"); return CPHNSW_B200_E_INVALID; }
    FileCloser fc{std::fopen(path, "wb")};
    if (!fc.f) { set_error("save: cannot create %s", path); return CPHNSW_B200_E_INVALID; }
    FileHeader hd{};
    hd.version = kFileVersion, hd.K = h->K, hd.comp_bytes = h->comp_bytes, hd.M = h->M, hd.ef_construction = h->ef_construction;
    hd.keep_pruned = uint32_t(h->keep_pruned), hd.k_entry = h->k_entry, hd.knn_k = h->knn_k, hd.entry_scan = h->entry_scan;
    hd.binary_codes = uint32_t(h->binary_codes);
    hd.residual = h->residual_bits | (h->residual_shift << 16);
    hd.convention = h->convention, hd.dim = h->dim, hd.seed = h->seed, hd.n = h->n, hd.calib_samples = h->calib_samples;
    hd.calib_alpha = h->calib_alpha, hd.calib_beta = h->calib_beta, hd.calib_r2 = h->calib_r2;
    bool ok = std::fwrite(kFileMagic, 1, 8, fc.f) == 8 && std::fwrite(&hd, sizeof(hd), 1, fc.f) == 1 &&
              std::fwrite(h->signs.data(), 1, h->signs.size(), fc.f) == h->signs.size();
    if (!ok) { set_error("save: write failed"); return CPHNSW_B200_E_INVALID; }
    std::vector<char> buf(size_t(64) << 20);
    if (h->n) {
        CPB_TRY(write_device(fc.f, h->d_vectors.p, h->n * h->dim * 4, buf));
        if (h->codes_released) {  // the file keeps one component per bit
            std::vector<unsigned char> codes(h->n * code_row_bytes(h));
            CPB_TRY(host_codes_from_packed(h, 0, h->n, codes.data()));
            if (std::fwrite(codes.data(), 1, codes.size(), fc.f) != codes.size()) { set_error("save: write failed"); return CPHNSW_B200_E_INVALID; }
        } else {
            CPB_TRY(write_device(fc.f, h->d_codes.p, h->n * code_row_bytes(h), buf));
        }
        CPB_TRY(write_device(fc.f, h->d_adj.p, h->n * h->M * 4, buf));
    }
    std::FILE* f = fc.f;
    fc.f = nullptr;
    if (std::fclose(f) != 0) { set_error("save: write failed"); return CPHNSW_B200_E_INVALID; }
    return 0;
}

int cphnsw_b200_load(const char* path, int device, cphnsw_b200_index** out) {
    if (!path || !out) { set_error("load: null argument"); return CPHNSW_B200_E_INVALID; }
    *out = nullptr;
    FileCloser fc{std::fopen(path, "rb")};
    if (!fc.f) { set_error("load: cannot open %s", path); return CPHNSW_B200_E_INVALID; }
    char magic[8];
    FileHeader hd{};
    if (std::fread(magic, 1, 8, fc.f) != 8 || std::memcmp(magic, kFileMagic, 8) != 0) {
        set_error("load: %s is not a cphnsw_b200 index file", path);
        return CPHNSW_B200_E_INVALID;
    }
    if (std::fread(&hd, sizeof(hd), 1, fc.f) != 1 || hd.version != kFileVersion) {
        set_error("load: unsupported index file version");
        return CPHNSW_B200_E_INVALID;
    }
    if (hd.n >= 0x80000000ull) { set_error("load: corrupt header (n)"); return CPHNSW_B200_E_INVALID; }
    // the payload the header promises must be what the file holds, before anything is allocated for it
    if (hd.dim == 0 || hd.dim > 65536 || hd.K == 0 || hd.K > 256 || (hd.comp_bytes != 1 && hd.comp_bytes != 2) || hd.M == 0 ||
        hd.M > 64) {
        set_error("load: corrupt header (shape)");
        return CPHNSW_B200_E_INVALID;
    }
    {
        const uint64_t P = next_pow2(hd.dim);
        const uint64_t want = 8 + sizeof(hd) + uint64_t(hd.K) * 3 * P +
                              hd.n * (hd.dim * 4 + uint64_t(hd.K) * hd.comp_bytes + uint64_t(hd.M) * 4);
        const long here = std::ftell(fc.f);
        if (here < 0 || std::fseek(fc.f, 0, SEEK_END) != 0) { set_error("load: cannot size %s", path); return CPHNSW_B200_E_INVALID; }
        const long size = std::ftell(fc.f);
        if (size < 0 || uint64_t(size) != want || std::fseek(fc.f, here, SEEK_SET) != 0) {
            set_error("load: %s holds %ld bytes, its header promises %llu", path, size, (unsigned long long)want);
            return CPHNSW_B200_E_INVALID;
        }
    }
    cphnsw_b200_index* h = nullptr;
    CPB_TRY(create_impl(hd.dim, hd.K, hd.comp_bytes, hd.M, hd.ef_construction, hd.seed, hd.convention, device,
                        hd.binary_codes != 0, &h));
    struct Guard {
        cphnsw_b200_index* h;
        ~Guard() { delete h; }
    } guard{h};
    std::vector<int8_t> signs(h->signs.size());
    if (std::fread(signs.data(), 1, signs.size(), fc.f) != signs.size()) { set_error("load: file is shorter than its header says"); return CPHNSW_B200_E_INVALID; }
    CPB_TRY(cphnsw_b200_set_sign_tables(h, signs.data()));
    if (hd.k_entry < 1 || hd.k_entry > 100 || hd.knn_k > 64 || hd.entry_scan > 1048576) { set_error("load: corrupt header (tunables)"); return CPHNSW_B200_E_INVALID; }
    h->binary_codes = hd.binary_codes != 0;
    {
        const uint32_t rb = hd.residual & 0xffffu, rs = hd.residual >> 16;
        if (rb >= hd.K || rs > 4 || (rb && (!hd.binary_codes || ((hd.K - rb) * hd.comp_bytes) % 4 != 0))) { set_error("load: corrupt header (residual codes)"); return CPHNSW_B200_E_INVALID; }
        h->residual_bits = rb, h->residual_shift = rs;
    }
    h->keep_pruned = hd.keep_pruned != 0, h->k_entry = hd.k_entry, h->knn_k = hd.knn_k, h->entry_scan = hd.entry_scan;
    h->calib_alpha = hd.calib_alpha, h->calib_beta = hd.calib_beta, h->calib_r2 = hd.calib_r2, h->calib_samples = hd.calib_samples;
    if (hd.n) {
        const uint64_t n = hd.n;
        CPB_TRY(h->d_vectors.reserve(n * h->dim * 4));
        CPB_TRY(h->d_codes.reserve(n * code_row_bytes(h) + 16));
        h->codes_released = false;
        CPB_TRY(h->d_adj.reserve(n * h->M * 4 + 16));
        std::vector<char> buf(size_t(64) << 20);
        CPB_TRY(read_device(fc.f, h->d_vectors.p, n * h->dim * 4, buf));
        CPB_TRY(read_device(fc.f, h->d_codes.p, n * code_row_bytes(h), buf));
        CPB_TRY(read_device(fc.f, h->d_adj.p, n * h->M * 4, buf));
        h->n = n;
        CPB_TRY(set_entry_ids(h));
    }
    guard.h = nullptr;
    *out = h;
    return 0;
}

// ---- host-pointer entry points -------------------------------------------------------------------------
int cphnsw_b200_encode(cphnsw_b200_index* h, const float* x, uint64_t n, void* codes_out) {
    return cphnsw_b200_encode_queries(h, x, n, codes_out, nullptr, nullptr);
}

int cphnsw_b200_encode_queries(cphnsw_b200_index* h, const float* q, uint64_t nq, void* codes_out, float* rotated_out,
                               float* magnitudes_out) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (nq == 0) return 0;
    if (!q || !codes_out) { set_error("encode: null pointer"); return CPHNSW_B200_E_INVALID; }
    const size_t rb = code_row_bytes(h);
    const size_t tf = size_t(h->K) * h->P;
    // bound the staging buffers: rotated output is K*P floats per row
    const uint64_t chunk = rotated_out ? 8192 : (uint64_t(1) << 22);
    for (uint64_t i0 = 0; i0 < nq; i0 += chunk) {
        const uint64_t m = nq - i0 < chunk ? nq - i0 : chunk;
        CPB_TRY(h->s_in.reserve(m * h->dim * 4));
        CPB_TRY(h->s_out.reserve(m * rb + 16));
        float *d_rot = nullptr, *d_mag = nullptr;
        if (rotated_out) { CPB_TRY(h->d_qtables.reserve(m * tf * 4)); d_rot = h->d_qtables.as<float>(); }
        if (magnitudes_out) { CPB_TRY(h->s_out2.reserve(m * h->K * 4)); d_mag = h->s_out2.as<float>(); }
        CPB_CUDA(cudaMemcpy(h->s_in.p, q + i0 * h->dim, m * h->dim * 4, cudaMemcpyHostToDevice));
        CPB_TRY(launch_encode(h, h->s_in.as<float>(), m, h->s_out.p, d_rot, d_mag, 0));
        CPB_CUDA(cudaMemcpy((char*)codes_out + i0 * rb, h->s_out.p, m * rb, cudaMemcpyDeviceToHost));
        if (rotated_out) CPB_CUDA(cudaMemcpy(rotated_out + i0 * tf, d_rot, m * tf * 4, cudaMemcpyDeviceToHost));
        if (magnitudes_out) CPB_CUDA(cudaMemcpy(magnitudes_out + i0 * h->K, d_mag, m * h->K * 4, cudaMemcpyDeviceToHost));
    }
    return 0;
}

int cphnsw_b200_code_distance(cphnsw_b200_index* h, const void* a, uint64_t na, const void* b, uint64_t nb,
                              uint16_t* out) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (na == 0 || nb == 0) return 0;
    if (!a || !b || !out) { set_error("code_distance: null pointer"); return CPHNSW_B200_E_INVALID; }
    const size_t rb = code_row_bytes(h);
    CPB_TRY(h->s_in.reserve(na * rb + 16));
    CPB_TRY(h->s_in2.reserve(nb * rb + 16));
    CPB_TRY(h->s_out.reserve(na * nb * 2));
    CPB_CUDA(cudaMemcpy(h->s_in.p, a, na * rb, cudaMemcpyHostToDevice));
    CPB_CUDA(cudaMemcpy(h->s_in2.p, b, nb * rb, cudaMemcpyHostToDevice));
    CPB_TRY(launch_code_distance(h, h->s_in.p, na, h->s_in2.p, nb, h->s_out.as<uint16_t>(), 0));
    CPB_CUDA(cudaMemcpy(out, h->s_out.p, na * nb * 2, cudaMemcpyDeviceToHost));
    return 0;
}

int cphnsw_b200_knn_graph(cphnsw_b200_index* h, const void* codes, uint64_t n, uint32_t k, uint64_t row_begin,
                          uint64_t row_end, uint32_t* nbrs_out, uint16_t* dist_out) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (row_end <= row_begin) return 0;
    if (!codes || !nbrs_out) { set_error("knn_graph: null pointer"); return CPHNSW_B200_E_INVALID; }
    const size_t rb = code_row_bytes(h);
    const uint64_t rows = row_end - row_begin;
    CPB_TRY(h->s_in.reserve(n * rb + 16));
    CPB_TRY(h->s_out.reserve(rows * k * 4));
    if (dist_out) CPB_TRY(h->s_out2.reserve(rows * k * 2));
    CPB_CUDA(cudaMemcpy(h->s_in.p, codes, n * rb, cudaMemcpyHostToDevice));
    CPB_TRY(launch_knn_graph(h, h->s_in.p, n, k, row_begin, row_end, h->s_out.as<uint32_t>(),
                             dist_out ? h->s_out2.as<uint16_t>() : nullptr, 0));
    CPB_CUDA(cudaMemcpy(nbrs_out, h->s_out.p, rows * k * 4, cudaMemcpyDeviceToHost));
    if (dist_out) CPB_CUDA(cudaMemcpy(dist_out, h->s_out2.p, rows * k * 2, cudaMemcpyDeviceToHost));
    return check_status(h);
}

int cphnsw_b200_select_neighbors(cphnsw_b200_index* h, const void* codes, uint64_t n, const uint32_t* cand, uint32_t k,
                                 uint64_t row_begin, uint64_t row_end, uint32_t M, int keep_pruned, uint32_t* adj_out) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (row_end <= row_begin) return 0;
    if (!codes || !cand || !adj_out) { set_error("select_neighbors: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (row_end > n) { set_error("select_neighbors: row range exceeds n"); return CPHNSW_B200_E_INVALID; }
    const size_t rb = code_row_bytes(h);
    const uint64_t rows = row_end - row_begin;
    CPB_TRY(h->s_in.reserve(n * rb + 16));
    CPB_TRY(h->s_in2.reserve(rows * k * 4));
    CPB_TRY(h->s_out.reserve(rows * M * 4));
    CPB_CUDA(cudaMemcpy(h->s_in.p, codes, n * rb, cudaMemcpyHostToDevice));
    CPB_CUDA(cudaMemcpy(h->s_in2.p, cand, rows * k * 4, cudaMemcpyHostToDevice));
    CPB_TRY(launch_select_neighbors(h, h->s_in.p, n, h->s_in2.as<uint32_t>(), k, row_begin, row_end, M, keep_pruned,
                                    h->s_out.as<uint32_t>(), 0));
    CPB_CUDA(cudaMemcpy(adj_out, h->s_out.p, rows * M * 4, cudaMemcpyDeviceToHost));
    return 0;
}

int cphnsw_b200_rank_prune(cphnsw_b200_index* h, const uint32_t* cand, uint64_t n, uint32_t k, uint32_t M, float alpha,
                           uint32_t* adj_out) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (n == 0) return 0;
    if (!cand || !adj_out) { set_error("rank_prune: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (!(alpha >= 1.0f) || alpha > 3.0f) { set_error("rank_prune: alpha must be in 1.0..3.0"); return CPHNSW_B200_E_INVALID; }
    CPB_TRY(h->s_in2.reserve(n * k * 4 + 16));
    CPB_TRY(h->s_out.reserve(n * M * 4 + 16));
    CPB_CUDA(cudaMemcpy(h->s_in2.p, cand, n * k * 4, cudaMemcpyHostToDevice));
    CPB_TRY(launch_rank_prune(h, n, h->s_in2.as<uint32_t>(), k, M, alpha, h->s_out.as<uint32_t>(), 0));
    CPB_CUDA(cudaMemcpy(adj_out, h->s_out.p, n * M * 4, cudaMemcpyDeviceToHost));
    return 0;
}

int cphnsw_b200_rank_reorder_dev(cphnsw_b200_index* h, const uint32_t* d_cand, uint64_t n, uint32_t k, uint64_t row_begin,
                                 uint64_t row_end, uint32_t M, float alpha, uint32_t* d_kept, void* stream) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (row_end > row_begin && (!d_cand || !d_kept)) { set_error("rank_reorder: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (!(alpha >= 1.0f) || alpha > 3.0f) { set_error("rank_reorder: alpha must be in 1.0..3.0"); return CPHNSW_B200_E_INVALID; }
    return launch_rank_reorder(h, n, d_cand, k, row_begin, row_end, M, alpha, d_kept, (cudaStream_t)stream);
}

int cphnsw_b200_rank_merge_dev(cphnsw_b200_index* h, const uint32_t* d_kept, uint64_t n, uint32_t M, uint64_t row_begin,
                               uint64_t row_end, uint32_t* d_adj, void* stream) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    if (row_end > row_begin && (!d_kept || !d_adj)) { set_error("rank_merge: null pointer"); return CPHNSW_B200_E_INVALID; }
    return launch_rank_merge(h, n, d_kept, M, row_begin, row_end, d_adj, (cudaStream_t)stream);
}

static int add_batch_impl(cphnsw_b200_index* h, const float* x, uint64_t n);

// callers hold the handle's lock exclusively
static int add_batch_parallel_impl(cphnsw_b200_index* h, const float* x, uint64_t n) {
    if (n == 0) return 0;
    if (!x) { set_error("add_batch_parallel: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (h->n + n >= 0x80000000ull) { set_error("add_batch_parallel: at most 2^31-1 nodes"); return CPHNSW_B200_E_INVALID; }
    if (h->build_seed && h->n == 0 && n > h->build_seed) {
        // the exact kNN graph of the first build_seed vectors, the others inserted into it
        const uint32_t seed_n = h->build_seed;
        h->build_seed = 0;
        int rc = add_batch_parallel_impl(h, x, seed_n);
        h->build_seed = seed_n;
        CPB_TRY(rc);
        return add_batch_impl(h, x + uint64_t(seed_n) * h->dim, n - seed_n);
    }
    // the new adjacency is built beside the old one and the handle (n, adjacency) changes only once
    // everything has succeeded: a failure on the way leaves the index as it was
    const uint64_t old_n = h->n, total = h->n + n;
    const size_t rb = code_row_bytes(h);
    CPB_TRY(ensure_codes(h, 0));
    CPB_TRY(grow_keep(h->d_vectors, old_n * h->dim * 4, total * h->dim * 4));
    CPB_TRY(grow_keep(h->d_codes, old_n * rb, total * rb + 16));
    float* d_new = h->d_vectors.as<float>() + old_n * h->dim;
    CPB_CUDA(cudaMemcpy(d_new, x, n * h->dim * 4, cudaMemcpyHostToDevice));
    CPB_TRY(launch_encode(h, d_new, n, h->d_codes.as<unsigned char>() + old_n * rb, nullptr, nullptr, 0));
    DevBuf adj;
    CPB_TRY(build_graph(h, total, adj, 0));
    h->d_adj.swap(adj);
    h->n = total;
    drop_search_scratch(h);  // visited arrays are sized by n
    return set_entry_ids(h);
}


int cphnsw_b200_add_batch_parallel(cphnsw_b200_index* h, const float* x, uint64_t n) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    return add_batch_parallel_impl(h, x, n);
}

int cphnsw_b200_add_batch(cphnsw_b200_index* h, const float* x, uint64_t n) {
    CPB_TRY(bind(h));
    std::unique_lock<std::shared_mutex> guard(h->rw);
    return add_batch_impl(h, x, n);
}

static int add_batch_impl(cphnsw_b200_index* h, const float* x, uint64_t n) {
    if (n == 0) return 0;
    if (!x) { set_error("add_batch: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (h->n == 0) return add_batch_parallel_impl(h, x, n);  // nothing to insert into: bulk build
    if (h->n + n >= 0x80000000ull) { set_error("add_batch: at most 2^31-1 nodes"); return CPHNSW_B200_E_INVALID; }
    const size_t rb = code_row_bytes(h);
    cudaStream_t st = 0;
    for (uint64_t done = 0; done < n;) {
        const uint64_t n_old = h->n;
        const uint64_t m = n - done < n_old ? n - done : n_old;  // a piece never outnumbers the graph it joins
        CPB_TRY(ensure_codes(h, st));
        CPB_TRY(grow_keep(h->d_vectors, n_old * h->dim * 4, (n_old + m) * h->dim * 4));
        CPB_TRY(grow_keep(h->d_codes, n_old * rb, (n_old + m) * rb + 16));
        CPB_TRY(grow_keep(h->d_adj, n_old * h->M * 4, (n_old + m) * h->M * 4 + 16));
        float* d_new = h->d_vectors.as<float>() + n_old * h->dim;
        unsigned char* d_new_codes = h->d_codes.as<unsigned char>() + n_old * rb;
        CPB_CUDA(cudaMemcpyAsync(d_new, x + done * h->dim, m * h->dim * 4, cudaMemcpyHostToDevice, st));
        CPB_TRY(launch_encode(h, d_new, m, d_new_codes, nullptr, nullptr, st));
        // candidates: a walk of the existing graph under the code distance from the usual seeds
        const uint32_t k_c = uint32_t(n_old < 64 ? n_old : 64);
        uint32_t beam = h->ef_construction > k_c ? h->ef_construction : k_c;
        if (beam > 1024) beam = 1024;
        CtxLease lease;
        CPB_TRY(lease.acquire(h, true));
        SearchCtx& cx = *lease.cx;
        CPB_TRY(lease.begin(st));
        CPB_TRY(cx.d_out_ids.reserve(m * k_c * 4));
        CPB_TRY(cx.d_out_dist.reserve(m * k_c * 4));
        CPB_TRY(launch_search(h, cx, nullptr, nullptr, m, k_c, beam, 0, cx.d_out_ids.as<uint32_t>(), cx.d_out_dist.as<float>(),
                              nullptr, st, d_new_codes));
        CPB_TRY(launch_select_neighbors(h, h->d_codes.p, n_old + m, cx.d_out_ids.as<uint32_t>(), k_c, n_old, n_old + m, h->M,
                                        h->keep_pruned, h->d_adj.as<uint32_t>() + n_old * h->M, st));
        CPB_TRY(launch_reverse_edges(h, h->d_codes.p, n_old, m, h->d_adj.as<uint32_t>(), h->M, h->keep_pruned, st));
        CPB_CUDA(cudaStreamSynchronize(st));
        CPB_TRY(check_status(h));
        h->n = n_old + m;
        CPB_TRY(set_entry_ids(h));
        done += m;
    }
    return 0;
}

int cphnsw_b200_get_codes(const cphnsw_b200_index* h, void* codes_out) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    if (!codes_out) { set_error("get_codes: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (h->n && h->codes_released) return host_codes_from_packed(h, 0, h->n, static_cast<unsigned char*>(codes_out));
    if (h->n) CPB_CUDA(cudaMemcpy(codes_out, h->d_codes.p, h->n * code_row_bytes(h), cudaMemcpyDeviceToHost));
    return 0;
}

int cphnsw_b200_get_adjacency(const cphnsw_b200_index* h, uint32_t* adj_out) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    if (!adj_out) { set_error("get_adjacency: null pointer"); return CPHNSW_B200_E_INVALID; }
    if (h->n) CPB_CUDA(cudaMemcpy(adj_out, h->d_adj.p, h->n * h->M * 4, cudaMemcpyDeviceToHost));
    return 0;
}

int cphnsw_b200_get_entry_ids(const cphnsw_b200_index* h, uint32_t* ids_out, uint64_t* count) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    if (count) *count = h->n_entry;
    if (ids_out && h->n_entry) CPB_CUDA(cudaMemcpy(ids_out, h->d_entry.p, size_t(h->n_entry) * 4, cudaMemcpyDeviceToHost));
    return 0;
}

int cphnsw_b200_search_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k, uint32_t ef,
                             uint32_t* ids_out, float* dists_out, uint32_t* stats_out) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    return do_search(h, q, false, nq, k, ef, 0, ids_out, dists_out, stats_out, false, 0);
}

int cphnsw_b200_search_multiprobe_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k, uint32_t ef,
                                        uint32_t num_probes, uint32_t* ids_out, float* dists_out) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    return do_multiprobe(h, q, nq, k, ef, num_probes, ids_out, dists_out, nullptr, true);
}

int cphnsw_b200_probe_codes(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t num_probes, void* codes_out) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    if (nq && !codes_out) { set_error("probe_codes: null output pointer"); return CPHNSW_B200_E_INVALID; }
    return do_multiprobe(h, q, nq, 1, 1, num_probes, nullptr, nullptr, codes_out, false);
}

int cphnsw_b200_search_and_rerank_batch(cphnsw_b200_index* h, const float* q, uint64_t nq, uint32_t k, uint32_t ef,
                                        uint32_t rerank_k, uint32_t* ids_out, float* dists_out, uint32_t* stats_out) {
    CPB_TRY(bind(h));
    std::shared_lock<std::shared_mutex> guard(h->rw);
    if (rerank_k == 0) { set_error("search_and_rerank: rerank_k must be > 0"); return CPHNSW_B200_E_INVALID; }
    return do_search(h, q, false, nq, k, ef, rerank_k, ids_out, dists_out, stats_out, false, 0);
}

}  // extern "C"
