// Cross-polytope encode: Psi(x) = H D3 H D2 H D1 x for K rotations, fused with the signed
// argmax that produces one code component per rotation.
//
// What it computes follows the reference's RandomHadamardRotation::apply_copy
// (include/cphnsw/encoder/rotation.hpp:90-111), fht (include/cphnsw/encoder/transform/fht.hpp),
// detail::find_argmax_abs (include/cphnsw/encoder/cp_encoder.hpp:25-92) and CPCode::encode
// (include/cphnsw/core/types.hpp:88-90).  Bit-exactness rests on three facts:
//   * every butterfly is one IEEE add or subtract in the stage order h = 1, 2, 4, ... — the
//     kernels use __fadd_rn/__fsub_rn (never contracted) in that order;
//   * multiplying by a +-1 diagonal is exact, so folding it into the first butterfly stage as
//     fma(s1, x1, s0*x0) rounds exactly like (s0*x0) + (s1*x1);
//   * the reference's SIMD FHT differs from its scalar FHT only by negating element i when
//     popcount(i & (W-1)) is odd (W = 8 AVX2, 16 AVX-512).  The host folds that diagonal into
//     the sign tables of layers 1 and 2; the last one only decides the sign bit of the code
//     (and the sign of the rotated output), applied here through `flip_mask` = W-1.
//
// Two kernels:
//   encode_p128_kernel   padded dim 128 (d in 65..128): one thread owns one vector, the whole
//                        128-point transform lives in registers (no shuffles, no barriers in the
//                        inner loop); the bound is the fp32 add pipe.
//   encode_warp_kernel   padded dims 32, 64, 256, 512: one warp per vector, P/32 consecutive elements per lane,
//                        low stages in registers, high stages by shuffles.
//   encode_generic_kernel any other power-of-two padded dim: one warp owns one vector in shared memory.
#include "common.cuh"

namespace cpb {
namespace {

constexpr int kP128 = 128;
constexpr int kTileVecs = 128;          // vectors per block = threads per block
// Padded row of the staged tile: thread t reads bank (t + i) & 31.  (Measured and dropped: a 132-float stride with
// 128-bit reloads, 3.875 ms per 1M vectors against 3.835 ms, and on top of it the diagonal applied as a sign-bit XOR
// on the integer pipe with plain first-stage butterflies, 3.883 ms.  Also measured and dropped: the diagonal folded
// into every stage - block multipliers t = s[i] * s[i + h], butterflies fma(+-t, y, x), one overall sign per layer
// left for the end - which is bit-equal and saves the 64 multiplies per layer, 3.894 ms: the three-operand
// instructions cost what the saved ones gave.)
constexpr int kTileStride = kP128 + 1;

template <int H>
__device__ __forceinline__ void butterfly_stage(float (&v)[kP128]) {
#pragma unroll
    for (int i = 0; i < kP128; i += 2 * H) {
#pragma unroll
        for (int j = i; j < i + H; ++j) {
            float x = v[j], y = v[j + H];
            v[j] = __fadd_rn(x, y);
            v[j + H] = __fsub_rn(x, y);
        }
    }
}

// D then H on 128 registers.  `sg` points at 128 +-1 floats in shared memory, read by every
// thread at the same address (broadcast).
__device__ __forceinline__ void diag_fht128(float (&v)[kP128], const float* __restrict__ sg) {
    const float4* s4 = reinterpret_cast<const float4*>(sg);
#pragma unroll
    for (int c = 0; c < kP128 / 4; ++c) {
        float4 s = s4[c];
        {
            float t = __fmul_rn(s.x, v[4 * c]);
            float y = v[4 * c + 1];
            v[4 * c] = __fmaf_rn(s.y, y, t);
            v[4 * c + 1] = __fmaf_rn(-s.y, y, t);
        }
        {
            float t = __fmul_rn(s.z, v[4 * c + 2]);
            float y = v[4 * c + 3];
            v[4 * c + 2] = __fmaf_rn(s.w, y, t);
            v[4 * c + 3] = __fmaf_rn(-s.w, y, t);
        }
    }
    butterfly_stage<2>(v);
    butterfly_stage<4>(v);
    butterfly_stage<8>(v);
    butterfly_stage<16>(v);
    butterfly_stage<32>(v);
    butterfly_stage<64>(v);
}

// Lowest-index argmax of |v| by a left-biased tournament: the right operand wins only when it is
// strictly larger, so among equal magnitudes the lowest index survives every round
// (same answer as the strict `>` scan of cp_encoder.hpp:82-88).
__device__ __forceinline__ void argmax128(const float (&v)[kP128], float& win, int& idx) {
    float w[64];
    int id[64];
#pragma unroll
    for (int j = 0; j < 64; ++j) {
        bool r = fabsf(v[2 * j + 1]) > fabsf(v[2 * j]);
        w[j] = r ? v[2 * j + 1] : v[2 * j];
        id[j] = r ? 2 * j + 1 : 2 * j;
    }
#pragma unroll
    for (int n = 32; n >= 1; n >>= 1) {
#pragma unroll
        for (int j = 0; j < n; ++j) {
            bool r = fabsf(w[2 * j + 1]) > fabsf(w[2 * j]);
            w[j] = r ? w[2 * j + 1] : w[2 * j];
            id[j] = r ? id[2 * j + 1] : id[2 * j];
        }
    }
    win = w[0];
    idx = id[0];
}

// sign bit of the component: `value < 0` (cp_encoder.hpp:174) after the convention's last
// diagonal, which negates the value when popcount(idx & flip_mask) is odd.
__device__ __forceinline__ uint32_t component_of(float win, int idx, int flip_mask) {
    bool flip = __popc(idx & flip_mask) & 1;
    bool neg = flip ? (win > 0.0f) : (win < 0.0f);
    return (uint32_t(idx) << 1) | (neg ? 1u : 0u);
}

// QUERY = true additionally writes the rotated vectors and winning magnitudes (CPQuery).
template <typename CompT, bool QUERY>
__global__ void __launch_bounds__(kTileVecs, QUERY ? 2 : 3)
encode_p128_kernel(const float* __restrict__ x, uint64_t n, int dim, int K,
                   const float* __restrict__ signs /*[K][3][128]*/, int flip_mask,
                   CompT* __restrict__ codes, float* __restrict__ rotated, float* __restrict__ mags) {
    extern __shared__ float smem[];
    float* tile = smem;                                                 // [kTileVecs][kTileStride]
    float* sign_sm = tile + kTileVecs * kTileStride;                              // [2][3][128], double buffer
    CompT* code_tile = reinterpret_cast<CompT*>(sign_sm + 2 * 3 * kP128);         // [kTileVecs][K]

    const uint64_t row0 = uint64_t(blockIdx.x) * kTileVecs;
    const int rows = int(min(uint64_t(kTileVecs), n - row0));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // stage the tile: coalesced 128-bit loads when rows are 16-byte aligned, else 32-bit loads
    const bool vec4 = (dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    for (int r = warp; r < kTileVecs; r += kTileVecs / 32) {
        float* dst = tile + r * kTileStride;
        if (r < rows) {
            const float* src = x + (row0 + r) * uint64_t(dim);
            if (vec4) {
                float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
                if (4 * lane < dim) q = __ldg(reinterpret_cast<const float4*>(src) + lane);
                dst[4 * lane] = q.x;
                dst[4 * lane + 1] = q.y;
                dst[4 * lane + 2] = q.z;
                dst[4 * lane + 3] = q.w;
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    int i = lane + 32 * c;
                    dst[i] = i < dim ? __ldg(src + i) : 0.0f;
                }
            }
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) dst[lane + 32 * c] = 0.0f;
        }
    }
    // the three diagonals of one rotation are staged in shared memory one rotation ahead
    const int t = threadIdx.x;
    if (t < 3 * kP128 / 4)
        reinterpret_cast<float4*>(sign_sm)[t] = __ldg(reinterpret_cast<const float4*>(signs) + t);
    __syncthreads();

    const float* mine = tile + t * kTileStride;
    const uint64_t row = row0 + t;
    for (int r = 0; r < K; ++r) {
        if (r + 1 < K && t < 3 * kP128 / 4)
            reinterpret_cast<float4*>(sign_sm + ((r + 1) & 1) * 3 * kP128)[t] =
                __ldg(reinterpret_cast<const float4*>(signs + size_t(r + 1) * 3 * kP128) + t);
        float v[kP128];
#pragma unroll
        for (int i = 0; i < kP128; ++i) v[i] = mine[i];
        const float* sg = sign_sm + (r & 1) * 3 * kP128;
#pragma unroll 1
        for (int layer = 0; layer < 3; ++layer) diag_fht128(v, sg + layer * kP128);
        float win;
        int idx;
        argmax128(v, win, idx);
        code_tile[t * K + r] = CompT(component_of(win, idx, flip_mask));
        if (QUERY && t < rows) {
            if (mags) mags[row * K + r] = fabsf(win);
            if (rotated) {
                float4* out = reinterpret_cast<float4*>(rotated + (row * K + r) * kP128);
#pragma unroll
                for (int c = 0; c < kP128 / 4; ++c) {
                    float4 o;
                    o.x = (__popc((4 * c) & flip_mask) & 1) ? -v[4 * c] : v[4 * c];
                    o.y = (__popc((4 * c + 1) & flip_mask) & 1) ? -v[4 * c + 1] : v[4 * c + 1];
                    o.z = (__popc((4 * c + 2) & flip_mask) & 1) ? -v[4 * c + 2] : v[4 * c + 2];
                    o.w = (__popc((4 * c + 3) & flip_mask) & 1) ? -v[4 * c + 3] : v[4 * c + 3];
                    out[c] = o;
                }
            }
        }
        __syncthreads();  // the next rotation's diagonals are in place, this rotation's are free
    }
    // the tile's codes are contiguous in the output: write them back coalesced
    const int total = rows * K;
    CompT* dst = codes + row0 * uint64_t(K);
    for (int i = threadIdx.x; i < total; i += kTileVecs) dst[i] = code_tile[i];
}

// ---- padded dim 1024 (d in 513..1024): one warp per vector, 32 elements per lane -------------------
// The 10 stages of a 1024-point transform are done as two register passes of a 32-point transform:
// stages h = 1..16 with the lane holding 32 consecutive elements (i = 32*lane + j), stages
// h = 32..512 with the lane holding a stride-32 column (i = 32*j + lane), and a transpose through a
// padded 32x33 shared-memory tile between the two layouts.  The stage order h = 1, 2, 4, ... and
// the butterfly (lo = x + y, hi = x - y, x the lower index) are the reference's, so the result is
// bit-identical.  The diagonals come bit-packed in the layout they are applied in (a set bit
// negates), one word per lane and layer.
constexpr int kP1024 = 1024;
constexpr int kWarps1024 = 4;

__device__ __forceinline__ void fht32_regs(float (&v)[32]) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if ((j & h) == 0) {
                const float x = v[j], y = v[j + h];
                v[j] = __fadd_rn(x, y);
                v[j + h] = __fsub_rn(x, y);
            }
        }
    }
}

__device__ __forceinline__ void flip_signs32(float (&v)[32], uint32_t word) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
        v[j] = __int_as_float(__float_as_int(v[j]) ^ int((word << (31 - j)) & 0x80000000u));
}

template <typename CompT, bool QUERY>
__global__ void __launch_bounds__(kWarps1024 * 32)
encode_p1024_kernel(const float* __restrict__ x, uint64_t n, int dim, int K,
                    const uint32_t* __restrict__ signbits /*[K][3][32]*/, int flip_mask,
                    CompT* __restrict__ codes, float* __restrict__ rotated, float* __restrict__ mags) {
    __shared__ float tiles[kWarps1024][32 * 33];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* buf = tiles[warp];
    const bool vec4 = (dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    for (uint64_t row = uint64_t(blockIdx.x) * kWarps1024 + warp; row < n; row += uint64_t(gridDim.x) * kWarps1024) {
        // the vector, zero-padded, in the consecutive layout: xin[j] = x[32*lane + j]
        float xin[32];
        const float* src = x + row * uint64_t(dim);
        if (vec4) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int i = 32 * lane + 4 * c;
                float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < dim) q = __ldg(reinterpret_cast<const float4*>(src + i));
                xin[4 * c] = q.x, xin[4 * c + 1] = q.y, xin[4 * c + 2] = q.z, xin[4 * c + 3] = q.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int i = 32 * lane + j;
                xin[j] = i < dim ? __ldg(src + i) : 0.0f;
            }
        }
        for (int r = 0; r < K; ++r) {
            const uint32_t* sb = signbits + size_t(r) * 3 * 32;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = xin[j];
#pragma unroll 1
            for (int layer = 0; layer < 3; ++layer) {
                const uint32_t word = __ldg(sb + layer * 32 + lane);
                flip_signs32(v, word);  // layer 0: consecutive layout; layers 1, 2: column layout
                if (layer > 0) {        // column -> consecutive
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 32; ++j) buf[j * 33 + lane] = v[j];
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = buf[lane * 33 + j];
                }
                fht32_regs(v);  // stages h = 1..16
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 32; ++j) buf[lane * 33 + j] = v[j];  // consecutive -> column
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = buf[j * 33 + lane];
                fht32_regs(v);  // stages h = 32..512
            }
            // column layout: v[j] is element 32*j + lane.  Lowest-index argmax of |v|.
            float best = -1.0f, win = 0.0f;
            int idx = 0x7fffffff;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float av = fabsf(v[j]);
                if (av > best) {
                    best = av;
                    win = v[j];
                    idx = 32 * j + lane;
                }
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const float ow = __shfl_xor_sync(0xffffffffu, win, o);
                const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
                if (ob > best || (ob == best && oi < idx)) {
                    best = ob;
                    win = ow;
                    idx = oi;
                }
            }
            if (lane == 0) {
                codes[row * K + r] = CompT(component_of(win, idx, flip_mask));
                if (QUERY && mags) mags[row * K + r] = best;
            }
            if (QUERY && rotated) {
                float* out = rotated + (row * K + r) * uint64_t(kP1024);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int i = 32 * j + lane;
                    out[i] = (__popc(i & flip_mask) & 1) ? -v[j] : v[j];
                }
            }
        }
    }
}

// ---- padded dims 32, 64, 256, 512: one warp per vector, E = P / 32 consecutive elements per lane -------------
// Lane L holds elements E*L .. E*L + E - 1.  Stages h < E pair elements of one lane (registers), stages
// h = E * 2^t pair lane L with lane L ^ 2^t (one shuffle per element): the lower index computes x + y, the upper
// x - y with x the lower element, in ascending h like the reference's loop (fht.hpp:56-69), so the result is
// bit-identical.  Nothing goes through shared memory.
template <typename CompT, bool QUERY, int E>
__global__ void __launch_bounds__(128)
encode_warp_kernel(const float* __restrict__ x, uint64_t n, int dim, int K, const float* __restrict__ signs /*[K][3][P]*/,
                   int flip_mask, CompT* __restrict__ codes, float* __restrict__ rotated, float* __restrict__ mags) {
    constexpr int P = 32 * E;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int first = E * lane;
    for (uint64_t row = uint64_t(blockIdx.x) * warps + warp; row < n; row += uint64_t(gridDim.x) * warps) {
        const float* src = x + row * uint64_t(dim);
        float in[E];
#pragma unroll
        for (int j = 0; j < E; ++j) in[j] = first + j < dim ? __ldg(src + first + j) : 0.0f;
        for (int r = 0; r < K; ++r) {
            float v[E];
#pragma unroll
            for (int j = 0; j < E; ++j) v[j] = in[j];
            const float* sg = signs + size_t(r) * 3 * P + first;
#pragma unroll 1
            for (int layer = 0; layer < 3; ++layer) {
#pragma unroll
                for (int j = 0; j < E; ++j) v[j] = __fmul_rn(v[j], __ldg(sg + layer * P + j));
#pragma unroll
                for (int h = 1; h < E; h <<= 1) {
#pragma unroll
                    for (int j = 0; j < E; ++j)
                        if ((j & h) == 0) {
                            const float a = v[j], b = v[j + h];
                            v[j] = __fadd_rn(a, b);
                            v[j + h] = __fsub_rn(a, b);
                        }
                }
#pragma unroll
                for (int t = 1; t < 32; t <<= 1) {
                    const bool upper = lane & t;
#pragma unroll
                    for (int j = 0; j < E; ++j) {
                        const float other = __shfl_xor_sync(0xffffffffu, v[j], t);
                        v[j] = upper ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
                    }
                }
            }
            // lowest-index argmax: ascending scan of the lane's own elements, then a warp reduction that prefers
            // the lower index on equal magnitude (cp_encoder.hpp:82-88)
            float best = -1.0f, win = 0.0f;
            int idx = 0x7fffffff;
#pragma unroll
            for (int j = 0; j < E; ++j) {
                const float a = fabsf(v[j]);
                if (a > best) {
                    best = a;
                    win = v[j];
                    idx = first + j;
                }
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const float ow = __shfl_xor_sync(0xffffffffu, win, o);
                const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
                if (ob > best || (ob == best && oi < idx)) {
                    best = ob;
                    win = ow;
                    idx = oi;
                }
            }
            if (lane == 0) {
                codes[row * K + r] = CompT(component_of(win, idx, flip_mask));
                if (QUERY && mags) mags[row * K + r] = best;
            }
            if (QUERY && rotated) {
                float* out = rotated + (row * K + r) * uint64_t(P) + first;
#pragma unroll
                for (int j = 0; j < E; ++j) out[j] = (__popc((first + j) & flip_mask) & 1) ? -v[j] : v[j];
            }
        }
    }
}

// ---- generic padded dim: one warp per vector, transform in shared memory ----------------------
template <typename CompT>
__global__ void encode_generic_kernel(const float* __restrict__ x, uint64_t n, int dim, int P, int K,
                                      const float* __restrict__ signs /*[K][3][P]*/, int flip_mask,
                                      CompT* __restrict__ codes, float* __restrict__ rotated,
                                      float* __restrict__ mags) {
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    float* buf = smem + size_t(warp) * P;
    for (uint64_t row = uint64_t(blockIdx.x) * warps + warp; row < n; row += uint64_t(gridDim.x) * warps) {
        const float* src = x + row * uint64_t(dim);
        for (int r = 0; r < K; ++r) {
            const float* sg = signs + size_t(r) * 3 * P;
            for (int layer = 0; layer < 3; ++layer) {
                // diagonal (layer 0 also loads and zero-pads)
                for (int i = lane; i < P; i += 32) {
                    float a = layer == 0 ? (i < dim ? __ldg(src + i) : 0.0f) : buf[i];
                    buf[i] = __fmul_rn(a, sg[layer * P + i]);
                }
                __syncwarp();
                for (int h = 1; h < P; h <<= 1) {
                    for (int b = lane; b < P / 2; b += 32) {
                        int j = ((b / h) * 2 * h) + (b % h);
                        float a = buf[j], c = buf[j + h];
                        buf[j] = __fadd_rn(a, c);
                        buf[j + h] = __fsub_rn(a, c);
                    }
                    __syncwarp();
                }
            }
            // lowest-index argmax: strided scan per lane (ascending index), then a warp
            // reduction that prefers the lower index on equal magnitude
            float best = -1.0f, win = 0.0f;  // -1: the first element a lane sees always wins
            int idx = 0x7fffffff;
            for (int i = lane; i < P; i += 32) {
                float a = fabsf(buf[i]);
                if (a > best) {
                    best = a;
                    win = buf[i];
                    idx = i;
                }
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                float ob = __shfl_xor_sync(0xffffffffu, best, o);
                float ow = __shfl_xor_sync(0xffffffffu, win, o);
                int oi = __shfl_xor_sync(0xffffffffu, idx, o);
                if (ob > best || (ob == best && oi < idx)) {
                    best = ob;
                    win = ow;
                    idx = oi;
                }
            }
            if (lane == 0) {
                codes[row * K + r] = CompT(component_of(win, idx, flip_mask));
                if (mags) mags[row * K + r] = best;
            }
            if (rotated) {
                float* out = rotated + (row * K + r) * uint64_t(P);
                for (int i = lane; i < P; i += 32)
                    out[i] = (__popc(i & flip_mask) & 1) ? -buf[i] : buf[i];
            }
            __syncwarp();
        }
    }
}

}  // namespace

// binary-code mode: every component reduced to its sign bit; 32-bit words where the buffer allows
__global__ void sign_only_kernel(uint32_t* __restrict__ codes, uint64_t words, uint32_t mask) {
    const uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < words) codes[i] &= mask;
}
__global__ void sign_only_bytes_kernel(unsigned char* __restrict__ codes, uint64_t bytes, int comp_bytes) {
    const uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < bytes) codes[i] &= (comp_bytes == 2 && (i & 1)) ? 0u : 1u;  // little-endian halfwords: the high byte is cleared
}

int launch_encode(cphnsw_b200_index* h, const float* d_x, uint64_t n, void* d_codes, float* d_rot,
                  float* d_mag, cudaStream_t st) {
    if (n == 0) return 0;
    const int P = int(h->P), K = int(h->K), dim = int(h->dim);
    // width of the reference's in-register SIMD phase for this build and length
    // (fht.hpp:141-147: AVX-512 defers to AVX2 below 16; :81-87: AVX2 defers to scalar below 8)
    int w = 1;
    if (h->convention == CPHNSW_B200_FHT_AVX512 && P >= 16) w = 16;
    else if (h->convention >= CPHNSW_B200_FHT_AVX2 && P >= 8) w = 8;
    const int flip_mask = w - 1;
    const float* signs = h->d_signs.as<float>();
    LaunchTimer timer(h, kKernelEncode, st);

    if (P == kP128) {
        size_t smem = size_t(kTileVecs) * kTileStride * sizeof(float) + size_t(2) * 3 * kP128 * sizeof(float) +
                      size_t(kTileVecs) * K * h->comp_bytes;
        unsigned grid = unsigned((n + kTileVecs - 1) / kTileVecs);
        const bool query = d_rot || d_mag;
#define CPB_LAUNCH_P128(T, Q)                                                                              \
    do {                                                                                                   \
        CPB_CUDA(allow_max_dynamic_smem(encode_p128_kernel<T, Q>));                                        \
        encode_p128_kernel<T, Q><<<grid, kTileVecs, smem, st>>>(d_x, n, dim, K, signs, flip_mask,           \
                                                               (T*)d_codes, d_rot, d_mag);                  \
    } while (0)
        if (h->comp_bytes == 1) {
            if (query) CPB_LAUNCH_P128(uint8_t, true);
            else CPB_LAUNCH_P128(uint8_t, false);
        } else {
            if (query) CPB_LAUNCH_P128(uint16_t, true);
            else CPB_LAUNCH_P128(uint16_t, false);
        }
#undef CPB_LAUNCH_P128
    } else if (P == kP1024 && h->d_signbits.p) {
        const bool query = d_rot || d_mag;
        const uint64_t blocks = (n + kWarps1024 - 1) / kWarps1024;
        const unsigned grid = unsigned(blocks < uint64_t(h->sm_count) * 16 ? blocks : uint64_t(h->sm_count) * 16);
        const uint32_t* sb = h->d_signbits.as<uint32_t>();
#define CPB_LAUNCH_P1024(T, Q)                                                                              \
    encode_p1024_kernel<T, Q><<<grid, kWarps1024 * 32, 0, st>>>(d_x, n, dim, K, sb, flip_mask, (T*)d_codes, d_rot, d_mag)
        if (h->comp_bytes == 1) {  // (a 1-byte component cannot hold a 1024-wide index; kept for symmetry)
            if (query) CPB_LAUNCH_P1024(uint8_t, true);
            else CPB_LAUNCH_P1024(uint8_t, false);
        } else {
            if (query) CPB_LAUNCH_P1024(uint16_t, true);
            else CPB_LAUNCH_P1024(uint16_t, false);
        }
#undef CPB_LAUNCH_P1024
    } else if (P == 32 || P == 64 || P == 256 || P == 512) {
        const bool query = d_rot || d_mag;
        const uint64_t blocks = (n + 3) / 4;
        const unsigned grid = unsigned(blocks < uint64_t(h->sm_count) * 32 ? blocks : uint64_t(h->sm_count) * 32);
#define CPB_LAUNCH_WARP(T, Q, EE) \
    encode_warp_kernel<T, Q, EE><<<grid, 128, 0, st>>>(d_x, n, dim, K, signs, flip_mask, (T*)d_codes, d_rot, d_mag)
#define CPB_LAUNCH_WARP_E(T, Q)                      \
    do {                                             \
        if (P == 32) CPB_LAUNCH_WARP(T, Q, 1);       \
        else if (P == 64) CPB_LAUNCH_WARP(T, Q, 2);  \
        else if (P == 256) CPB_LAUNCH_WARP(T, Q, 8); \
        else CPB_LAUNCH_WARP(T, Q, 16);              \
    } while (0)
        if (h->comp_bytes == 1) {
            if (query) CPB_LAUNCH_WARP_E(uint8_t, true);
            else CPB_LAUNCH_WARP_E(uint8_t, false);
        } else {
            if (query) CPB_LAUNCH_WARP_E(uint16_t, true);
            else CPB_LAUNCH_WARP_E(uint16_t, false);
        }
#undef CPB_LAUNCH_WARP_E
#undef CPB_LAUNCH_WARP
    } else {
        int warps = 4;
        while (warps > 1 && size_t(warps) * P * sizeof(float) > 96 * 1024) warps >>= 1;
        size_t smem = size_t(warps) * P * sizeof(float);
        uint64_t blocks = (n + warps - 1) / warps;
        unsigned grid = unsigned(blocks < uint64_t(h->sm_count) * 16 ? blocks : uint64_t(h->sm_count) * 16);
        if (h->comp_bytes == 1) {
            CPB_CUDA(allow_max_dynamic_smem(encode_generic_kernel<uint8_t>));
            encode_generic_kernel<uint8_t><<<grid, warps * 32, smem, st>>>(d_x, n, dim, P, K, signs, flip_mask,
                                                                          (uint8_t*)d_codes, d_rot, d_mag);
        } else {
            CPB_CUDA(allow_max_dynamic_smem(encode_generic_kernel<uint16_t>));
            encode_generic_kernel<uint16_t><<<grid, warps * 32, smem, st>>>(d_x, n, dim, P, K, signs, flip_mask,
                                                                           (uint16_t*)d_codes, d_rot, d_mag);
        }
    }
    h->launches++;
    CPB_CUDA(cudaGetLastError());
    if (h->binary_codes && d_codes) {
        // binary-code mode: a component keeps only its sign bit (the unified encoder's primary code,
        // include/cphnsw/encoder/cp_encoder.hpp:165-176)
        const uint64_t bytes = n * uint64_t(K) * h->comp_bytes;
        if ((reinterpret_cast<uintptr_t>(d_codes) & 3) == 0 && (bytes & 3) == 0)
            sign_only_kernel<<<unsigned((bytes / 4 + 255) / 256), 256, 0, st>>>(static_cast<uint32_t*>(d_codes), bytes / 4,
                                                                              h->comp_bytes == 2 ? 0x00010001u : 0x01010101u);
        else
            sign_only_bytes_kernel<<<unsigned((bytes + 255) / 256), 256, 0, st>>>(static_cast<unsigned char*>(d_codes), bytes,
                                                                                 int(h->comp_bytes));
        h->launches++;
        CPB_CUDA(cudaGetLastError());
    }
    return 0;
}

}  // namespace cpb
