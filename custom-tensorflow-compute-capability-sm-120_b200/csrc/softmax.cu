// Row softmax for the attention path of the matmul op on B200: the step between
// the two batched GEMMs (Q.K^T and P.V) when attention is NOT run as one fused
// kernel (a mask, returned attention weights, fp32 tensors), and the standalone
// softmax launcher.
//
// Replaces sm120_softmax_kernel (src/cuda_kernels/sm120_pure_kernels.cu:471-550,
// launched by src/cuda_kernels/sm120_c_interface.cu:374-400): the same result,
// softmax over `axis_size` with fp32 math and a max subtraction.  The reference
// reads every logit three times with one block per (outer, inner) pair and two
// shared-memory tree reductions; here a row that fits in registers (up to 8192
// elements) is read ONCE with 16-byte loads by one warp, reduced with shuffles and
// written once, so the kernel is bound by HBM bandwidth (one read + one write).
// Longer rows, and softmax over a strided axis (inner_size > 1), take a block-per-row
// three-pass path.
//
// The extended form folds in what the attention layer applies before the softmax
// (python/sm120_ops.py:385-402, python/sm120_keras_layers.py:815-822): a scale, an
// additive mask (times a factor, -1e9 in the layer) and the causal mask.

#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "gemm_common.h"

namespace sm120 {

struct SoftmaxParams {
    const void* in;
    void* out;
    long long rows, cols;
    float scale;                 // logits are multiplied by it first
    const float* mask;           // null, or additive mask of mask_rows x cols floats, row r uses mask row r % mask_rows
    long long mask_rows;
    float mask_factor;           // the mask is multiplied by it (1, or -1e9 for a 0/1 "masked" indicator)
    int causal;                  // column c of row r is dropped when c > (r % seq_q) + cols - seq_q
    long long seq_q;
};

template <typename T> __device__ __forceinline__ float sm_to_float(T v);
template <> __device__ __forceinline__ float sm_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float sm_to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float sm_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T sm_from_float(float v);
template <> __device__ __forceinline__ float sm_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half sm_from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 sm_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// fp32 tensors keep expf; 16-bit results have at most 11 significand bits, for which the
// hardware exponential (relative error ~1e-6) is exact after rounding
template <typename T> __device__ __forceinline__ float sm_exp(float x) {
    if constexpr (sizeof(T) == 4) return expf(x);
    else return __expf(x);
}

__device__ __forceinline__ float logit_of(const SoftmaxParams& p, float raw, long long row, long long col) {
    float v = raw * p.scale;
    if (p.mask != nullptr) v = fmaf(p.mask_factor, __ldg(p.mask + (row % p.mask_rows) * p.cols + col), v);
    if (p.causal && col > (row % p.seq_q) + p.cols - p.seq_q) v = -CUDART_INF_F;
    return v;
}

constexpr int SM_WARPS = 8;

// One warp per row; NV 16-byte vectors per lane hold the whole row (cols <= 32 * VEC * NV, cols % VEC == 0,
// rows 16-byte aligned).  The grid is persistent (a few CTAs per SM) and every warp walks over rows
// row, row + W, ...: the raw vectors of its NEXT row are requested before the current row is reduced, so
// loads are in flight all the time instead of only at the start of a short-lived CTA.
// TO is T, or a 16-bit type when T is float (fp32 scores in, 16-bit probabilities out for the P.V product).
// PLAIN: no mask and no causal cut (the per-element tests of the masked form are compiled out: fully unrolled
// they make the kernel so large that it stalls on instruction fetch).
template <typename T, typename TO, int NV, bool PLAIN>
__global__ void __launch_bounds__(32 * SM_WARPS)
sm120_softmax_rows_kernel(const SoftmaxParams p) {
    constexpr int VEC = 16 / sizeof(T);
    const int lane = threadIdx.x & 31;
    const long long nwarps = static_cast<long long>(gridDim.x) * SM_WARPS;
    const long long nvec = p.cols / VEC;
    long long row = static_cast<long long>(blockIdx.x) * SM_WARPS + (threadIdx.x >> 5);
    uint4 raw[NV];
    if (row < p.rows) {
        const uint4* in = reinterpret_cast<const uint4*>(static_cast<const T*>(p.in) + row * p.cols);
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (lane + 32ll * i < nvec) raw[i] = __ldcs(in + lane + 32 * i);
    }
    for (; row < p.rows; row += nwarps) {
        float v[NV][VEC];
        float m = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const long long iv = lane + 32ll * i;
            if (iv < nvec) {
                const T* e = reinterpret_cast<const T*>(&raw[i]);
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    if constexpr (PLAIN) v[i][k] = sm_to_float<T>(e[k]) * p.scale;
                    else v[i][k] = logit_of(p, sm_to_float<T>(e[k]), row, iv * VEC + k);
                    m = fmaxf(m, v[i][k]);
                }
            }
        }
        // the next row's vectors travel while this row is reduced and written
        const long long next = row + nwarps;
        if (next < p.rows) {
            const uint4* in = reinterpret_cast<const uint4*>(static_cast<const T*>(p.in) + next * p.cols);
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (lane + 32ll * i < nvec) raw[i] = __ldcs(in + lane + 32 * i);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        if (m == -CUDART_INF_F) m = 0.0f;              // a fully masked row: every exponential is 0, handled below
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (lane + 32ll * i < nvec) {
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    v[i][k] = sm_exp<TO>(v[i][k] - m);
                    s += v[i][k];
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        const float inv = s > 0.0f ? 1.0f / s : 0.0f;
        TO* out = static_cast<TO*>(p.out) + row * p.cols;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const long long iv = lane + 32ll * i;
            if (iv < nvec) {
                if constexpr (sizeof(TO) == sizeof(T)) {
                    uint4 w;
                    TO* e = reinterpret_cast<TO*>(&w);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) e[k] = sm_from_float<TO>(v[i][k] * inv);
                    __stcs(reinterpret_cast<uint4*>(out) + iv, w);
                } else {                                    // four fp32 in, four 16-bit values (8 bytes) out
                    uint2 w;
                    TO* e = reinterpret_cast<TO*>(&w);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) e[k] = sm_from_float<TO>(v[i][k] * inv);
                    __stcs(reinterpret_cast<uint2*>(out) + iv, w);
                }
            }
        }
    }
}

// General path: one block per (outer, inner) pair, softmax over `axis` elements `inner` apart; three passes.
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
sm120_softmax_strided_kernel(const SoftmaxParams p, long long axis, long long inner) {
    __shared__ float red[32];
    const long long outer_idx = blockIdx.x / inner, inner_idx = blockIdx.x % inner;
    const long long row = blockIdx.x;                        // for masks (inner == 1): the row number
    const T* in = static_cast<const T*>(p.in) + outer_idx * axis * inner + inner_idx;
    TO* out = static_cast<TO*>(p.out) + outer_idx * axis * inner + inner_idx;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    auto block_reduce = [&](float x, bool is_max) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float y = __shfl_xor_sync(0xFFFFFFFFu, x, o);
            x = is_max ? fmaxf(x, y) : x + y;
        }
        __syncthreads();
        if (lane == 0) red[warp] = x;
        __syncthreads();
        x = red[0];
        for (int w = 1; w < 8; ++w) x = is_max ? fmaxf(x, red[w]) : x + red[w];     // fixed order
        return x;
    };
    float m = -CUDART_INF_F;
    for (long long i = threadIdx.x; i < axis; i += 256) m = fmaxf(m, logit_of(p, sm_to_float<T>(in[i * inner]), row, i));
    m = block_reduce(m, true);
    if (m == -CUDART_INF_F) m = 0.0f;
    float s = 0.0f;
    for (long long i = threadIdx.x; i < axis; i += 256) s += sm_exp<TO>(logit_of(p, sm_to_float<T>(in[i * inner]), row, i) - m);
    s = block_reduce(s, false);
    const float inv = s > 0.0f ? 1.0f / s : 0.0f;
    for (long long i = threadIdx.x; i < axis; i += 256)
        out[i * inner] = sm_from_float<TO>(sm_exp<TO>(logit_of(p, sm_to_float<T>(in[i * inner]), row, i) - m) * inv);
}

template <typename T, typename TO>
static cudaError_t softmax_typed(const SoftmaxParams& p, long long outer, long long axis, long long inner, int sm_count, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = (reinterpret_cast<uintptr_t>(p.in) & 15u) == 0 &&
                         (reinterpret_cast<uintptr_t>(p.out) & (VEC * sizeof(TO) - 1)) == 0;
    if (inner == 1 && aligned && axis % VEC == 0 && axis <= 32ll * VEC * 16) {
        const long long nvec = axis / VEC;
        long long blocks = (outer + SM_WARPS - 1) / SM_WARPS;
        const long long cap = static_cast<long long>(sm_count) * 4;       // persistent: the kernel strides over the rows
        if (blocks > cap) blocks = cap;
        const unsigned grid = static_cast<unsigned>(blocks);
        const bool plain = p.mask == nullptr && !p.causal;
#define SM120_SOFTMAX_ROWS(NV_)                                                                                   \
    do {                                                                                                          \
        if (plain) sm120_softmax_rows_kernel<T, TO, NV_, true><<<grid, 32 * SM_WARPS, 0, stream>>>(p);            \
        else sm120_softmax_rows_kernel<T, TO, NV_, false><<<grid, 32 * SM_WARPS, 0, stream>>>(p);                 \
    } while (0)
        if (nvec <= 32)       SM120_SOFTMAX_ROWS(1);
        else if (nvec <= 64)  SM120_SOFTMAX_ROWS(2);
        else if (nvec <= 128) SM120_SOFTMAX_ROWS(4);
        else if (nvec <= 256) SM120_SOFTMAX_ROWS(8);
        else                  SM120_SOFTMAX_ROWS(16);
#undef SM120_SOFTMAX_ROWS
        return cudaGetLastError();
    }
    const long long blocks = outer * inner;
    if (blocks > 0x7FFFFFFFll) return cudaErrorInvalidValue;
    sm120_softmax_strided_kernel<T, TO><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p, axis, inner);
    return cudaGetLastError();
}

// Softmax over the middle extent of [outer, axis, inner]; mask / causal need inner == 1.
// out_dtype is dtype, or a 16-bit type for fp32 logits.
cudaError_t softmax_launch(const void* in, void* out, long long outer, long long axis, long long inner, int dtype, int out_dtype,
                           float scale, const float* mask, long long mask_rows, float mask_factor, int causal, long long seq_q,
                           int sm_count, cudaStream_t stream) {
    SoftmaxParams p{};
    p.in = in; p.out = out;
    p.rows = outer * inner; p.cols = axis;
    p.scale = scale;
    p.mask = mask; p.mask_rows = mask_rows > 0 ? mask_rows : 1; p.mask_factor = mask_factor;
    p.causal = causal; p.seq_q = seq_q > 0 ? seq_q : 1;
    if (dtype == SM120_DTYPE_FLOAT32 && out_dtype == SM120_DTYPE_FLOAT16) return softmax_typed<float, __half>(p, outer, axis, inner, sm_count, stream);
    if (dtype == SM120_DTYPE_FLOAT32 && out_dtype == SM120_DTYPE_BFLOAT16) return softmax_typed<float, __nv_bfloat16>(p, outer, axis, inner, sm_count, stream);
    if (dtype != out_dtype) return cudaErrorInvalidValue;
    switch (dtype) {
        case SM120_DTYPE_FLOAT32:  return softmax_typed<float, float>(p, outer, axis, inner, sm_count, stream);
        case SM120_DTYPE_FLOAT16:  return softmax_typed<__half, __half>(p, outer, axis, inner, sm_count, stream);
        case SM120_DTYPE_BFLOAT16: return softmax_typed<__nv_bfloat16, __nv_bfloat16>(p, outer, axis, inner, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace sm120
