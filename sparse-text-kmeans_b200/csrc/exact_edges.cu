// Graph links chosen on the stored fp32 vectors instead of the codes: the legacy index's "hybrid" construction
// ("Hybrid (True Cosine edges) - the production path", evaluation/eval_master.cpp:251-272; evaluation/test_tiered.cpp:4-7;
// source absent).  Candidates of a node are its exact nearest neighbours by -<x,y>; select_neighbors
// (resources/hnsw-paper/consolidated.tex:93-115, keepPrunedConnections) then runs on those exact distances.
// Every distance is the CPU loop's float: products and sums separate, summed in d order.
#include "common.cuh"

namespace cpb {
namespace {

constexpr uint32_t kFull = 0xffffffffu;
constexpr int kMaxCand = 64;

// ids [rows][k + 1] from the exact search of the rows against all vectors (a row finds itself, normally first)
// -> cand [rows][k]: the list without the row's own id; when the row is not in its list (more than k exact
// duplicates with lower ids) the last entry is dropped instead.
__global__ void drop_self_kernel(const uint32_t* __restrict__ ids, uint64_t rows, uint64_t row_begin, uint32_t k,
                                 uint32_t* __restrict__ cand) {
    const uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows) return;
    const uint32_t self = uint32_t(row_begin + i);
    const uint32_t* in = ids + i * (k + 1);
    uint32_t* out = cand + i * k;
    uint32_t o = 0;
    for (uint32_t t = 0; t < k + 1 && o < k; ++t)
        if (in[t] != self) out[o++] = in[t];
}

__device__ __forceinline__ float neg_dot(const float* a, const float* b, int dim) {
    float acc = 0.0f;
    for (int d = 0; d < dim; ++d) acc = __fadd_rn(acc, __fmul_rn(a[d], b[d]));
    return -acc;
}

// One warp per node (one block per warp: the candidates' vectors fill its shared memory).  Candidate t is kept
// iff it is closer to the node than to every member kept so far; member m is tested by lane m % 32.
// SMEM = false reads the vectors from global memory (dimensions whose candidate set does not fit).
template <bool SMEM>
__global__ void __launch_bounds__(32)
select_exact_kernel(const float* __restrict__ vectors, uint64_t n, int dim, const uint32_t* __restrict__ cand, uint32_t k,
                    uint64_t row_begin, uint64_t row_end, uint32_t M, int keep_pruned, uint32_t* __restrict__ adj) {
    extern __shared__ float xs[];  // [k][dim + 1] candidate vectors, then the node's own [dim]
    __shared__ uint32_t cid[kMaxCand];
    const int lane = threadIdx.x;
    const uint64_t row = row_begin + blockIdx.x;
    if (row >= row_end) return;
    const int stride = dim + 1;  // lanes reading different rows at the same d hit different banks
    const uint32_t* crow = cand + (row - row_begin) * uint64_t(k);
    for (uint32_t t = lane; t < kMaxCand; t += 32) {
        uint32_t c = t < k ? crow[t] : kInvalidNode;
        cid[t] = c < n ? c : kInvalidNode;
    }
    __syncwarp();
    const float* own_g = vectors + row * uint64_t(dim);
    float* own = xs + size_t(k) * stride;
    if (SMEM) {
        for (uint32_t t = 0; t < k; ++t) {
            if (cid[t] == kInvalidNode) continue;
            const float* src = vectors + uint64_t(cid[t]) * dim;
            for (int d = lane; d < dim; d += 32) xs[size_t(t) * stride + d] = __ldg(src + d);
        }
        for (int d = lane; d < dim; d += 32) own[d] = __ldg(own_g + d);
        __syncwarp();
    }
    auto vec = [&](uint32_t t) -> const float* { return SMEM ? xs + size_t(t) * stride : vectors + uint64_t(cid[t]) * dim; };
    const float* q = SMEM ? own : own_g;
    uint32_t kept_t[2] = {kInvalidNode, kInvalidNode};  // candidate position of member lane + 32 * s
    uint32_t rsize = 0;
    unsigned long long kept = 0, disc = 0;
    for (uint32_t t = 0; t < k && rsize < M; ++t) {
        if (cid[t] == kInvalidNode) continue;
        const float* e = vec(t);
        float d_eq = 0.0f;
        if (lane == 0) d_eq = neg_dot(e, q, dim);
        d_eq = __shfl_sync(kFull, d_eq, 0);
        bool viol = false;
#pragma unroll
        for (int s = 0; s < 2; ++s)
            if (uint32_t(lane + 32 * s) < rsize) viol |= !(d_eq < neg_dot(e, vec(kept_t[s]), dim));
        if (__any_sync(kFull, viol)) {
            disc |= 1ull << t;
        } else {
            kept |= 1ull << t;
#pragma unroll
            for (int s = 0; s < 2; ++s)
                if (uint32_t(lane + 32 * s) == rsize) kept_t[s] = t;
            ++rsize;
        }
    }
    uint32_t* out = adj + (row - row_begin) * uint64_t(M);
    const uint32_t n_disc = keep_pruned ? uint32_t(__popcll(disc)) : 0u;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        const int t = lane + 32 * s;
        const unsigned long long below = (1ull << t) - 1ull;
        uint32_t pos = kInvalidNode;
        if ((kept >> t) & 1ull) pos = uint32_t(__popcll(kept & below));
        else if (keep_pruned && ((disc >> t) & 1ull)) pos = rsize + uint32_t(__popcll(disc & below));
        if (pos < M) out[pos] = cid[t];
    }
    const uint32_t total = min(M, rsize + n_disc);
    for (uint32_t o = total + lane; o < M; o += 32) out[o] = kInvalidNode;
}

}  // namespace

// exact candidates of rows [row_begin, row_end): d_cand uint32[rows][k]
int launch_exact_candidates(cphnsw_b200_index* h, const float* d_vectors, uint64_t n, uint32_t k, uint64_t row_begin,
                            uint64_t row_end, uint32_t* d_cand, cudaStream_t st) {
    if (row_end <= row_begin) return 0;
    if (k == 0 || k > kMaxCand) {
        set_error("exact candidates: k must be in 1..64 (got %u)", k);
        return CPHNSW_B200_E_INVALID;
    }
    const uint64_t chunk = 1u << 16;  // rows per exact search: bounds the (k + 1)-wide scratch
    CPB_TRY(h->s_in2.reserve(size_t(chunk) * (k + 1) * 4 + 16));
    CPB_TRY(h->s_out2.reserve(size_t(chunk) * (k + 1) * 4 + 16));
    for (uint64_t r0 = row_begin; r0 < row_end; r0 += chunk) {
        const uint64_t rows = row_end - r0 < chunk ? row_end - r0 : chunk;
        CPB_TRY(launch_exact_search(h, d_vectors, n, d_vectors + r0 * h->dim, rows, k + 1, h->s_in2.as<uint32_t>(),
                                    h->s_out2.as<float>(), st));
        drop_self_kernel<<<unsigned((rows + 255) / 256), 256, 0, st>>>(h->s_in2.as<uint32_t>(), rows, r0, k,
                                                                       d_cand + (r0 - row_begin) * uint64_t(k));
        h->launches++;
        CPB_CUDA(cudaGetLastError());
    }
    return 0;
}

int launch_select_exact(cphnsw_b200_index* h, const float* d_vectors, uint64_t n, const uint32_t* d_cand, uint32_t k,
                        uint64_t row_begin, uint64_t row_end, uint32_t M, int keep_pruned, uint32_t* d_adj, cudaStream_t st) {
    if (row_end <= row_begin) return 0;
    if (k == 0 || k > kMaxCand || M == 0 || M > 64) {
        set_error("select_neighbors (exact distances): need 1 <= k <= 64 and 1 <= M <= 64 (got k=%u M=%u)", k, M);
        return CPHNSW_B200_E_INVALID;
    }
    const int dim = int(h->dim);
    const size_t smem = (size_t(k) * (dim + 1) + dim) * sizeof(float);
    const unsigned grid = unsigned(row_end - row_begin);
    LaunchTimer timer(h, kKernelSelect, st);
    if (smem <= 200 * 1024) {
        CPB_CUDA(allow_max_dynamic_smem(select_exact_kernel<true>));
        select_exact_kernel<true><<<grid, 32, smem, st>>>(d_vectors, n, dim, d_cand, k, row_begin, row_end, M, keep_pruned, d_adj);
    } else {
        select_exact_kernel<false><<<grid, 32, 0, st>>>(d_vectors, n, dim, d_cand, k, row_begin, row_end, M, keep_pruned, d_adj);
    }
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace cpb
