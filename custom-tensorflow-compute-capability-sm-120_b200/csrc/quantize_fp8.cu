// Per-tensor FP8 (e4m3) quantisation for the FP8 matmul path:
//     scale = 448 / max|x|          (1 when the tensor is all zeros)
//     q[i]  = saturate_e4m3(x[i] * scale)       round-to-nearest-even, finite
// Non-finite input: an infinity counts as the largest finite float when the
// maximum is taken (the scale stays positive and finite; the infinity itself
// saturates to +-448, everything finite becomes 0); a NaN does not take part in
// the maximum and is written as the e4m3 NaN.
// The reference declares the type and the conversion
// (src/cuda_kernels/sm120_datatype_support.h:71-82,168-171;
// python/sm120_datatype_manager.py:88-98) but has no kernel that produces FP8
// operands; the matmul consumes `scale` through SM120GemmDesc::scale_a_dev /
// scale_b_dev, so no host round trip is needed between the two.
//
// Two launches on the caller's stream, both HBM-bound (x is read twice, q
// written once):
//   1. amax_partial : one block per span of 65536 elements -> partial[b] = max|x| of the span
//   2. scale_cast   : every block reduces the partials to the same maximum (block 0 writes *scale_out),
//                     then q = sat(x * scale), 16-byte loads where alignment allows, the spans in
//                     reverse order so that what the first pass read last is still in the L2
// `partial` is scratch memory: one float per span.  Every slot that a call reads
// is written by that call's first launch, so nothing has to be zero beforehand.

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <atomic>

#include "gemm_common.h"

namespace sm120 {

constexpr int64_t QUANT_SPAN = 65536;       // elements per partial maximum
constexpr int QUANT_THREADS = 256;

template <typename T> __device__ __forceinline__ float q_to_float(T v);
template <> __device__ __forceinline__ float q_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float q_to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float q_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < (blockDim.x >> 5) ? red[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
        if (lane == 0) red[0] = v;
    }
    __syncthreads();
    return red[0];
}

template <typename T>
__global__ void __launch_bounds__(QUANT_THREADS)
sm120_quant_amax_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partial) {
    __shared__ float red[32];
    constexpr int VEC = 16 / sizeof(T);
    const long long begin = static_cast<long long>(blockIdx.x) * QUANT_SPAN;
    const long long end = min(n, begin + QUANT_SPAN);
    float m = 0.0f;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;     // spans start at multiples of 65536 elements
    if (vec_ok) {
        const long long nvec = (end - begin) / VEC;
        const uint4* xv = reinterpret_cast<const uint4*>(x + begin);
        long long i = threadIdx.x;
        for (; i + 3 * QUANT_THREADS < nvec; i += 4 * QUANT_THREADS) {          // four loads in flight per thread
            uint4 w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) w[u] = __ldg(xv + i + u * QUANT_THREADS);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const T* e = reinterpret_cast<const T*>(&w[u]);
#pragma unroll
                for (int k = 0; k < VEC; ++k) m = fmaxf(m, fabsf(q_to_float<T>(e[k])));
            }
        }
        for (; i < nvec; i += QUANT_THREADS) {
            const uint4 w = __ldg(xv + i);
            const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
            for (int k = 0; k < VEC; ++k) m = fmaxf(m, fabsf(q_to_float<T>(e[k])));
        }
        for (long long i = begin + nvec * VEC + threadIdx.x; i < end; i += QUANT_THREADS) m = fmaxf(m, fabsf(q_to_float<T>(x[i])));
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += QUANT_THREADS) m = fmaxf(m, fabsf(q_to_float<T>(x[i])));
    }
    m = block_max(m, red);
    if (threadIdx.x == 0) partial[blockIdx.x] = m;
}

__device__ __forceinline__ uint8_t to_e4m3(float v) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

// q = sat_e4m3(x * scale).  FROM_PARTIALS: the scale is not given but derived here, by every CTA alike, from the
// partial maxima of the first kernel (the same reduction in the same order in every CTA, so all use the same bits;
// CTA 0 also writes it to `scale`); that saves a one-CTA kernel between the two passes over x.  The spans are walked
// from the last to the first: the first pass read x front to back, so its tail is what the L2 still holds.
template <typename T, bool FROM_PARTIALS>
__global__ void __launch_bounds__(QUANT_THREADS)
sm120_quant_scale_cast_kernel(const T* __restrict__ x, long long n, float* __restrict__ scale, uint8_t* __restrict__ q,
                              const float* __restrict__ partial, int nparts) {
    constexpr int VEC = 16 / sizeof(T);          // elements per 16-byte load
    float s;
    if constexpr (FROM_PARTIALS) {
        __shared__ float red[32];
        float m = 0.0f;
        for (int i = threadIdx.x; i < nparts; i += QUANT_THREADS) m = fmaxf(m, partial[i]);
        m = block_max(m, red);
        s = m > 0.0f ? 448.0f / fminf(m, 3.402823466e38f) : 1.0f;
        if (blockIdx.x == 0 && threadIdx.x == 0) *scale = s;
    } else {
        s = __ldg(scale);
    }
    const long long begin = static_cast<long long>(gridDim.x - 1 - blockIdx.x) * QUANT_SPAN;
    const long long end = min(n, begin + QUANT_SPAN);
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(q) & 15u) == 0;
    if (vec_ok) {
        const long long nvec = (end - begin) / VEC;
        const uint4* xv = reinterpret_cast<const uint4*>(x + begin);
        const auto cast_store = [&](const uint4& w, long long i) {
            const T* e = reinterpret_cast<const T*>(&w);
            uint8_t out[VEC];
#pragma unroll
            for (int k = 0; k < VEC; ++k) out[k] = to_e4m3(q_to_float<T>(e[k]) * s);
            uint8_t* dst = q + begin + i * VEC;
            if constexpr (VEC == 8) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(out);
            else *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(out);
        };
        long long i = threadIdx.x;
        for (; i + 3 * QUANT_THREADS < nvec; i += 4 * QUANT_THREADS) {          // four loads in flight per thread
            uint4 w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) w[u] = __ldcs(xv + i + u * QUANT_THREADS);          // last use of x
#pragma unroll
            for (int u = 0; u < 4; ++u) cast_store(w[u], i + u * QUANT_THREADS);
        }
        for (; i < nvec; i += QUANT_THREADS) cast_store(__ldcs(xv + i), i);
        for (long long i = begin + nvec * VEC + threadIdx.x; i < end; i += QUANT_THREADS) q[i] = to_e4m3(q_to_float<T>(x[i]) * s);
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += QUANT_THREADS) q[i] = to_e4m3(q_to_float<T>(x[i]) * s);
    }
}

long long quant_spans(long long n) { return (n + QUANT_SPAN - 1) / QUANT_SPAN; }

template <typename T>
static cudaError_t quant_typed(const void* x, long long n, uint8_t* q, float* scale_out, float* partial, cudaStream_t stream) {
    const long long spans = quant_spans(n);
    const T* xt = static_cast<const T*>(x);
    sm120_quant_amax_partial_kernel<T><<<static_cast<unsigned>(spans), QUANT_THREADS, 0, stream>>>(xt, n, partial);
    sm120_quant_scale_cast_kernel<T, true><<<static_cast<unsigned>(spans), QUANT_THREADS, 0, stream>>>(xt, n, scale_out, q, partial,
                                                                                                       static_cast<int>(spans));
    return cudaGetLastError();
}

// Enqueue the two kernels (partial maxima; final maximum + scale + cast).  `partial` must hold quant_spans(n) floats.
cudaError_t quant_launch(const void* x, int x_dtype, void* q, float* scale_out, long long n, float* partial, cudaStream_t stream) {
    if (quant_spans(n) > 0x7FFFFFFFll) return cudaErrorInvalidValue;
    switch (x_dtype) {
        case SM120_DTYPE_FLOAT32:  return quant_typed<float>(x, n, static_cast<uint8_t*>(q), scale_out, partial, stream);
        case SM120_DTYPE_FLOAT16:  return quant_typed<__half>(x, n, static_cast<uint8_t*>(q), scale_out, partial, stream);
        case SM120_DTYPE_BFLOAT16: return quant_typed<__nv_bfloat16>(x, n, static_cast<uint8_t*>(q), scale_out, partial, stream);
        default: return cudaErrorInvalidValue;
    }
}

// Only the third kernel, with a scale the caller already has (e.g. from the amax of a
// tensor that is sharded over several GPUs).
cudaError_t quant_cast_launch(const void* x, int x_dtype, void* q, const float* scale, long long n, cudaStream_t stream) {
    const long long spans = quant_spans(n);
    if (spans > 0x7FFFFFFFll) return cudaErrorInvalidValue;
    uint8_t* qq = static_cast<uint8_t*>(q);
    const unsigned grid = static_cast<unsigned>(spans);
    switch (x_dtype) {
        case SM120_DTYPE_FLOAT32:
            sm120_quant_scale_cast_kernel<float, false><<<grid, QUANT_THREADS, 0, stream>>>(static_cast<const float*>(x), n, const_cast<float*>(scale), qq, nullptr, 0);
            break;
        case SM120_DTYPE_FLOAT16:
            sm120_quant_scale_cast_kernel<__half, false><<<grid, QUANT_THREADS, 0, stream>>>(static_cast<const __half*>(x), n, const_cast<float*>(scale), qq, nullptr, 0);
            break;
        case SM120_DTYPE_BFLOAT16:
            sm120_quant_scale_cast_kernel<__nv_bfloat16, false><<<grid, QUANT_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), n, const_cast<float*>(scale), qq, nullptr, 0);
            break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Variant that allocates nothing: the partial maxima live in a fixed array in
// this library's own device image.
// ---------------------------------------------------------------------------
// Every GPU that loads the library holds these 16 KB until the process exits.
// One float per 65536-element span: 4096 spans cover 268 435 456 elements.
static __device__ __align__(256) float g_quant_static_partial[SM120_QUANTIZE_FP8_STATIC_MAX_ELEMENTS / QUANT_SPAN];

// In host code the array's name is only a handle: the device address has to be
// asked for, once per device and with that device current.
static std::atomic<float*> g_quant_static_addr[64];

cudaError_t quant_launch_static(const void* x, int x_dtype, void* q, float* scale_out, long long n, int device,
                                cudaStream_t stream) {
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    float* partial = g_quant_static_addr[device].load(std::memory_order_acquire);
    if (partial == nullptr) {
        void* addr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&addr, g_quant_static_partial);
        if (e != cudaSuccess) return e;
        if (addr == nullptr) return cudaErrorInvalidSymbol;
        partial = static_cast<float*>(addr);
        g_quant_static_addr[device].store(partial, std::memory_order_release);
    }
    return quant_launch(x, x_dtype, q, scale_out, n, partial, stream);
}

}  // namespace sm120
