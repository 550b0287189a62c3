// HBM-bound companions of the matmul op on B200:
//   * the standalone activation launcher (what is left of the Dense path when an
//     activation cannot be fused into the GEMM epilogue), optionally with a bias
//     add in the same pass;
//   * the bias gradient of the Dense layer: column sums of dC.
//
// sm120_activation_kernel replaces the reference kernel of the same purpose
// (src/cuda_kernels/sm120_pure_kernels.cu:128-176, launched by
// src/cuda_kernels/sm120_c_interface.cu:139-164 and used by the SM120FusedActivation
// op, src/tensorflow_ops/sm120_ops.cc:251-326): same formulas and codes, fp32 math,
// round-to-nearest cast back; an unknown code leaves the value unchanged, as the
// reference's `default:` does.  Where the reference runs one element per thread
// of a 1024-thread block, this kernel moves 16 bytes per load, keeps four loads
// in flight per thread and sizes its grid from the SM count, which is what a
// kernel needs to come near HBM bandwidth on this part.
//
// The bias gradient has no kernel of its own in the reference: its Dense layer
// adds the bias with tf.nn.bias_add (python/sm120_keras_layers.py:169), whose
// gradient is the column sum; the matmul gradients are
// src/tensorflow_ops/sm120_gradients.cc:22-212.

#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_common.h"

namespace sm120 {

constexpr int EW_THREADS = 256;
constexpr int EW_UNROLL = 4;          // 16-byte loads in flight per thread

template <typename T> __device__ __forceinline__ float ew_to_float(T v);
template <> __device__ __forceinline__ float ew_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float ew_to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float ew_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T ew_from_float(float v);
template <> __device__ __forceinline__ float ew_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half ew_from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 ew_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// out[i] = act(in[i] + bias[i % cols]) over n elements; bias may be null (then cols is unused).
// The vector path needs in/out 16-byte aligned and, with a bias, cols a multiple of the
// vector length (so a vector never straddles a row); the launcher checks and passes vec = 0 otherwise.
template <typename T, typename TB>
__global__ void __launch_bounds__(EW_THREADS)
sm120_activation_kernel(const T* __restrict__ in, T* __restrict__ out, long long n, const TB* __restrict__ bias, long long cols,
                        int act, int vec) {
    constexpr int VEC = 16 / sizeof(T);
    const long long tid = static_cast<long long>(blockIdx.x) * EW_THREADS + threadIdx.x;
    const long long nthreads = static_cast<long long>(gridDim.x) * EW_THREADS;
    long long done = 0;
    if (vec) {
        const long long nvec = n / VEC;
        const uint4* iv = reinterpret_cast<const uint4*>(in);
        uint4* ov = reinterpret_cast<uint4*>(out);
        // column of a vector's first element, carried along instead of divided out per vector:
        // consecutive vectors of a thread are nthreads * VEC elements apart
        const long long col_step = bias != nullptr ? (nthreads * VEC) % cols : 0;
        long long col = bias != nullptr ? (tid * VEC) % cols : 0;
        for (long long base = tid; base < nvec; base += nthreads * EW_UNROLL) {
            uint4 w[EW_UNROLL];
#pragma unroll
            for (int u = 0; u < EW_UNROLL; ++u) {
                const long long i = base + u * nthreads;
                if (i < nvec) w[u] = __ldcs(iv + i);          // streamed once: do not keep in L2
            }
#pragma unroll
            for (int u = 0; u < EW_UNROLL; ++u) {
                const long long i = base + u * nthreads;
                const long long col0 = col;
                col += col_step;
                if (col >= cols) col -= cols;
                if (i >= nvec) continue;
                T* e = reinterpret_cast<T*>(&w[u]);
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    float x = ew_to_float<T>(e[k]);
                    if (bias != nullptr) x += ew_to_float<TB>(__ldg(bias + col0 + k));
                    e[k] = ew_from_float<T>(apply_activation(x, act));
                }
                __stcs(ov + i, w[u]);
            }
        }
        done = nvec * VEC;
    }
    for (long long i = done + tid; i < n; i += nthreads) {
        float x = ew_to_float<T>(in[i]);
        if (bias != nullptr) x += ew_to_float<TB>(bias[i % cols]);
        out[i] = ew_from_float<T>(apply_activation(x, act));
    }
}

template <typename T, typename TB>
static cudaError_t act_launch_typed(const void* in, void* out, long long n, const void* bias, long long cols, int act,
                                    int sm_count, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const int vec = (aligned && (bias == nullptr || cols % VEC == 0)) ? 1 : 0;
    const long long per_block = static_cast<long long>(EW_THREADS) * EW_UNROLL * VEC;
    long long blocks = (n + per_block - 1) / per_block;
    const long long cap = static_cast<long long>(sm_count) * 8;        // 8 resident blocks of 256 threads per SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    sm120_activation_kernel<T, TB><<<static_cast<unsigned>(blocks), EW_THREADS, 0, stream>>>(
        static_cast<const T*>(in), static_cast<T*>(out), n, static_cast<const TB*>(bias), cols, act, vec);
    return cudaGetLastError();
}

template <typename T>
static cudaError_t act_launch_bias(const void* in, void* out, long long n, const void* bias, int bias_dtype, long long cols,
                                   int act, int sm_count, cudaStream_t stream) {
    if (bias == nullptr) return act_launch_typed<T, float>(in, out, n, nullptr, 1, act, sm_count, stream);
    switch (bias_dtype) {
        case SM120_DTYPE_FLOAT32:  return act_launch_typed<T, float>(in, out, n, bias, cols, act, sm_count, stream);
        case SM120_DTYPE_FLOAT16:  return act_launch_typed<T, __half>(in, out, n, bias, cols, act, sm_count, stream);
        case SM120_DTYPE_BFLOAT16: return act_launch_typed<T, __nv_bfloat16>(in, out, n, bias, cols, act, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t activation_launch(const void* in, void* out, long long n, const void* bias, int bias_dtype, long long cols,
                              int act, int dtype, int sm_count, cudaStream_t stream) {
    switch (dtype) {
        case SM120_DTYPE_FLOAT32:  return act_launch_bias<float>(in, out, n, bias, bias_dtype, cols, act, sm_count, stream);
        case SM120_DTYPE_FLOAT16:  return act_launch_bias<__half>(in, out, n, bias, bias_dtype, cols, act, sm_count, stream);
        case SM120_DTYPE_BFLOAT16: return act_launch_bias<__nv_bfloat16>(in, out, n, bias, bias_dtype, cols, act, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

// ---------------------------------------------------------------------------
// Bias gradient: grad_bias[n] = sum over m of grad_c[m, n], fp32 accumulation in a
// fixed order (bitwise reproducible, no atomics, no scratch memory).
// One block owns a strip of STRIP columns for all rows.  A strip row is STRIP * sizeof(T)
// contiguous bytes, fetched by LANES threads with one 16-byte load each; the block's 256
// threads therefore cover 256 / LANES rows per step, each thread keeps 16 / sizeof(T) fp32
// partial sums, and the row groups are added in shared memory at the end.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
sm120_bias_grad_kernel(const T* __restrict__ g, long long M, long long N, long long ld, float* __restrict__ out_f32,
                       T* __restrict__ out_t, int vec) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int LANES = 8;                        // threads per strip row
    constexpr int STRIP = LANES * VEC;              // columns per block: 32 fp32 or 64 16-bit
    constexpr int ROWS = EW_THREADS / LANES;        // 32 rows per step
    __shared__ float part[ROWS][STRIP + 1];
    const int lane = threadIdx.x % LANES;
    const int rgrp = threadIdx.x / LANES;
    const long long col0 = static_cast<long long>(blockIdx.x) * STRIP + lane * VEC;
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = 0.0f;
    if (vec && col0 + VEC <= N) {
        long long m = rgrp;
        for (; m + 7 * ROWS < M; m += 8 * ROWS) {                      // eight rows in flight per thread
            uint4 w[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) w[u] = __ldcs(reinterpret_cast<const uint4*>(g + (m + u * ROWS) * ld + col0));
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const T* e = reinterpret_cast<const T*>(&w[u]);
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k] += ew_to_float<T>(e[k]);
            }
        }
        for (; m < M; m += ROWS) {
            const uint4 w = __ldcs(reinterpret_cast<const uint4*>(g + m * ld + col0));
            const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k] += ew_to_float<T>(e[k]);
        }
    } else {
        for (long long m = rgrp; m < M; m += ROWS) {
#pragma unroll
            for (int k = 0; k < VEC; ++k)
                if (col0 + k < N) acc[k] += ew_to_float<T>(g[m * ld + col0 + k]);
        }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) part[rgrp][lane * VEC + k] = acc[k];
    __syncthreads();
    if (threadIdx.x < STRIP) {
        const long long col = static_cast<long long>(blockIdx.x) * STRIP + threadIdx.x;
        if (col < N) {
            float s = 0.0f;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) s += part[r][threadIdx.x];
            if (out_f32 != nullptr) out_f32[col] = s;
            else out_t[col] = ew_from_float<T>(s);
        }
    }
}

template <typename T>
static cudaError_t bias_grad_typed(const void* g, long long M, long long N, long long ld, void* out, int out_dtype, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int STRIP = 8 * VEC;
    const int vec = ((reinterpret_cast<uintptr_t>(g) & 15u) == 0 && (ld * sizeof(T)) % 16 == 0) ? 1 : 0;
    const long long blocks = (N + STRIP - 1) / STRIP;
    if (blocks > 0x7FFFFFFFll) return cudaErrorInvalidValue;
    float* of = out_dtype == SM120_DTYPE_FLOAT32 ? static_cast<float*>(out) : nullptr;
    T* ot = out_dtype == SM120_DTYPE_FLOAT32 ? nullptr : static_cast<T*>(out);
    sm120_bias_grad_kernel<T><<<static_cast<unsigned>(blocks), EW_THREADS, 0, stream>>>(static_cast<const T*>(g), M, N, ld, of, ot, vec);
    return cudaGetLastError();
}

// out_dtype is FLOAT32 or the input dtype.
cudaError_t bias_grad_launch(const void* g, int dtype, long long M, long long N, long long ld, void* out, int out_dtype,
                             cudaStream_t stream) {
    if (out_dtype != SM120_DTYPE_FLOAT32 && out_dtype != dtype) return cudaErrorInvalidValue;
    switch (dtype) {
        case SM120_DTYPE_FLOAT32:  return bias_grad_typed<float>(g, M, N, ld, out, out_dtype, stream);
        case SM120_DTYPE_FLOAT16:  return bias_grad_typed<__half>(g, M, N, ld, out, out_dtype, stream);
        case SM120_DTYPE_BFLOAT16: return bias_grad_typed<__nv_bfloat16>(g, M, N, ld, out, out_dtype, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace sm120
