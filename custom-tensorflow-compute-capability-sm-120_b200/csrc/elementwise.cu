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

// Activation of VEC values with the switch outside the element loop (one formula's code runs per
// vector).  FAST16: the result will be rounded to a 16-bit type (8 or 11 significand bits), so the
// exponential-based forms with the hardware exponential and reciprocal (relative error ~1e-6) are
// exact after rounding in all but a vanishing fraction of cases, and an order of magnitude cheaper
// than tanhf / expf / logf: without them the transcendental activations are bound by the SM's
// instruction rate instead of HBM.  fp32 tensors keep the accurate functions.
__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// Two fp32 values in one 64-bit register pair and sm_100's packed fp32 arithmetic on them (one issue slot for two
// results): the sigmoid-based 16-bit activations are bound by the instruction rate, not by HBM, without it.
__device__ __forceinline__ uint64_t ew_pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void ew_split2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t ew_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t ew_mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t ew_add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// 1 / (1 + 2^z) for a pair: sigmoid(t) with z = -t log2(e).  2^z = inf gives 0, 2^z = 0 gives 1.
__device__ __forceinline__ uint64_t ew_sigmoid_exp2_2(uint64_t z2) {
    float z0, z1, e0, e1, r0, r1, d0, d1;
    ew_split2(z2, z0, z1);
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(z0));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(z1));
    ew_split2(ew_add2(ew_pack2(e0, e1), ew_pack2(1.0f, 1.0f)), d0, d1);
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(d0));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(d1));
    return ew_pack2(r0, r1);
}

template <int VEC, bool FAST16>
__device__ __forceinline__ void activate_vec(float (&x)[VEC], int act) {
    if constexpr (!FAST16) {
        switch (act) {
#define SM120_ACT_CASE(CODE) case CODE: _Pragma("unroll") for (int k = 0; k < VEC; ++k) x[k] = apply_activation(x[k], CODE); break;
            SM120_ACT_CASE(SM120_ACTIVATION_RELU) SM120_ACT_CASE(SM120_ACTIVATION_LEAKY_RELU) SM120_ACT_CASE(SM120_ACTIVATION_ELU)
            SM120_ACT_CASE(SM120_ACTIVATION_SELU) SM120_ACT_CASE(SM120_ACTIVATION_GELU) SM120_ACT_CASE(SM120_ACTIVATION_SWISH)
            SM120_ACT_CASE(SM120_ACTIVATION_MISH) SM120_ACT_CASE(SM120_ACTIVATION_TANH) SM120_ACT_CASE(SM120_ACTIVATION_SIGMOID)
            SM120_ACT_CASE(SM120_ACTIVATION_GELU_ERF)
#undef SM120_ACT_CASE
            default: break;
        }
    } else {
        switch (act) {
            case SM120_ACTIVATION_RELU:
#pragma unroll
                for (int k = 0; k < VEC; ++k) x[k] = fmaxf(0.0f, x[k]);
                break;
            case SM120_ACTIVATION_LEAKY_RELU:
#pragma unroll
                for (int k = 0; k < VEC; ++k) x[k] = x[k] > 0.0f ? x[k] : 0.01f * x[k];
                break;
            case SM120_ACTIVATION_ELU:
#pragma unroll
                for (int k = 0; k < VEC; ++k) x[k] = x[k] > 0.0f ? x[k] : (__expf(x[k]) - 1.0f);
                break;
            case SM120_ACTIVATION_SELU:
#pragma unroll
                for (int k = 0; k < VEC; ++k) x[k] = x[k] > 0.0f ? 1.0507f * x[k] : 1.0507f * 1.67326f * (__expf(x[k]) - 1.0f);
                break;
            case SM120_ACTIVATION_GELU: {      // 0.5 x (1 + tanh(u)) = x sigmoid(2u), u = 0.79788 (x + 0.044715 x^3)
                if constexpr (VEC % 2 == 0) {
                    const uint64_t c3 = ew_pack2(0.044715f, 0.044715f), one = ew_pack2(1.0f, 1.0f);
                    const uint64_t cz = ew_pack2(-2.0f * 0.7978845608f * 1.4426950409f, -2.0f * 0.7978845608f * 1.4426950409f);
#pragma unroll
                    for (int k = 0; k < VEC; k += 2) {
                        const uint64_t x2 = ew_pack2(x[k], x[k + 1]);
                        const uint64_t t = ew_mul2(ew_fma2(ew_mul2(x2, x2), c3, one), x2);         // x + 0.044715 x^3
                        ew_split2(ew_mul2(x2, ew_sigmoid_exp2_2(ew_mul2(t, cz))), x[k], x[k + 1]);
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < VEC; ++k) {
                        const float u = 0.7978845608f * (x[k] + 0.044715f * x[k] * x[k] * x[k]);
                        x[k] = x[k] * fast_sigmoid(2.0f * u);
                    }
                }
                break;
            }
            case SM120_ACTIVATION_SWISH: {
                if constexpr (VEC % 2 == 0) {
                    const uint64_t cz = ew_pack2(-1.4426950409f, -1.4426950409f);
#pragma unroll
                    for (int k = 0; k < VEC; k += 2) {
                        const uint64_t x2 = ew_pack2(x[k], x[k + 1]);
                        ew_split2(ew_mul2(x2, ew_sigmoid_exp2_2(ew_mul2(x2, cz))), x[k], x[k + 1]);
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < VEC; ++k) x[k] = x[k] * fast_sigmoid(x[k]);
                }
                break;
            }
            case SM120_ACTIVATION_MISH:        // tanh(log(1 + e^x)) = n / (n + 2) with n = e^x (e^x + 2)
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    const float w = __expf(fminf(x[k], 20.0f));
                    const float n = w * (w + 2.0f);
                    x[k] = x[k] * __fdividef(n, n + 2.0f);
                }
                break;
            case SM120_ACTIVATION_TANH:        // tanh(x) = 2 sigmoid(2x) - 1
#pragma unroll
                for (int k = 0; k < VEC; ++k) x[k] = fmaf(2.0f, fast_sigmoid(2.0f * x[k]), -1.0f);
                break;
            case SM120_ACTIVATION_SIGMOID:
#pragma unroll
                for (int k = 0; k < VEC; ++k) x[k] = fast_sigmoid(x[k]);
                break;
            case SM120_ACTIVATION_GELU_ERF:    // Abramowitz-Stegun 7.1.26 erf, |error| <= 1.5e-7
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    const float z = x[k] * 0.70710678118654752440f;
                    const float az = fabsf(z);
                    const float t = __fdividef(1.0f, fmaf(0.3275911f, az, 1.0f));
                    float poly = 1.061405429f;
                    poly = fmaf(poly, t, -1.453152027f);
                    poly = fmaf(poly, t, 1.421413741f);
                    poly = fmaf(poly, t, -0.284496736f);
                    poly = fmaf(poly, t, 0.254829592f);
                    poly *= t;
                    const float erf_abs = fmaf(-poly, __expf(-az * az), 1.0f);
                    x[k] = 0.5f * x[k] * (1.0f + copysignf(erf_abs, z));
                }
                break;
            default: break;
        }
    }
}

// out[i] = act(in[i] + bias[i % cols]) over n elements; bias may be null (then cols is unused).
// The vector path needs in/out 16-byte aligned and, with a bias, cols a multiple of the
// vector length (so a vector never straddles a row); the launcher checks and passes vec = 0 otherwise.
template <typename T, typename TB>
__global__ void __launch_bounds__(EW_THREADS, 5)      // 48 registers: five blocks per SM measured best (4.0 -> 5.2 TB/s on one box)
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
                float x[VEC];
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    x[k] = ew_to_float<T>(e[k]);
                    if (bias != nullptr) x[k] += ew_to_float<TB>(__ldg(bias + col0 + k));
                }
                activate_vec<VEC, sizeof(T) == 2>(x, act);
#pragma unroll
                for (int k = 0; k < VEC; ++k) e[k] = ew_from_float<T>(x[k]);
                __stcs(ov + i, w[u]);
            }
        }
        done = nvec * VEC;
    }
    for (long long i = done + tid; i < n; i += nthreads) {
        float x[1] = {ew_to_float<T>(in[i])};
        if (bias != nullptr) x[0] += ew_to_float<TB>(bias[i % cols]);
        activate_vec<1, sizeof(T) == 2>(x, act);
        out[i] = ew_from_float<T>(x[0]);
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
    const long long cap = static_cast<long long>(sm_count) * 5;        // the five resident blocks per SM: one wave (8 per SM: 5.2 instead of 5.4 TB/s)
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
// A thread-block CLUSTER of up to 8 CTAs owns a strip of STRIP columns: CTA r of the
// cluster sums the rows r * M / csize .. (r + 1) * M / csize of the strip, the partial sums
// meet in distributed shared memory, and CTA 0 adds them in rank order and writes the
// result.  The row split is what puts enough CTAs (strips x 8) and loads in flight to
// approach HBM bandwidth on a matrix with few column strips; the fixed order keeps it
// deterministic.  Inside a CTA a strip row is STRIP * sizeof(T) contiguous bytes fetched by
// LANES threads with one 16-byte load each; the 256 threads cover 256 / LANES rows per step.
// LANES = 32 (512 contiguous bytes per row and CTA) is what HBM likes best (5.4 TB/s on bf16 [8192, 11008] against
// 4.6 with 128-byte pieces); narrower strips are chosen only when the wide ones would leave the GPU short of CTAs.
// ---------------------------------------------------------------------------
constexpr int BG_MAX_CLUSTER = 8;
constexpr long long BG_MIN_CTAS = 256;            // below this many CTAs a narrower strip is tried

__device__ __forceinline__ uint32_t bg_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t bg_cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}

template <typename T, int BG_LANES>
__global__ void __launch_bounds__(EW_THREADS)
sm120_bias_grad_kernel(const T* __restrict__ g, long long M, long long N, long long ld, float* __restrict__ out_f32,
                       T* __restrict__ out_t, int vec) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int BG_ROWS = EW_THREADS / BG_LANES;  // rows per step
    constexpr int STRIP = BG_LANES * VEC;           // columns per cluster
    static_assert(STRIP <= EW_THREADS, "one thread per strip column in the final sums");
    __shared__ float part[BG_ROWS][STRIP + 1];
    __shared__ float strip_sum[STRIP];              // this CTA's partial column sums, read by CTA 0 of the cluster
    const uint32_t crank = bg_cluster_rank(), csize = bg_cluster_size();
    const int lane = threadIdx.x % BG_LANES;
    const int rgrp = threadIdx.x / BG_LANES;
    const long long col0 = static_cast<long long>(blockIdx.x) * STRIP + lane * VEC;
    // this CTA's rows: a contiguous share, in whole steps of BG_ROWS
    const long long steps = (M + BG_ROWS - 1) / BG_ROWS;
    const long long m_begin = (steps * crank / csize) * BG_ROWS;
    const long long m_end = min(M, (steps * (crank + 1) / csize) * BG_ROWS);
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = 0.0f;
    if (vec && col0 + VEC <= N) {
        long long m = m_begin + rgrp;
        for (; m + 7 * BG_ROWS < m_end; m += 8 * BG_ROWS) {                      // eight rows in flight per thread
            uint4 w[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) w[u] = __ldcs(reinterpret_cast<const uint4*>(g + (m + u * BG_ROWS) * ld + col0));
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const T* e = reinterpret_cast<const T*>(&w[u]);
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k] += ew_to_float<T>(e[k]);
            }
        }
        for (; m < m_end; m += BG_ROWS) {
            const uint4 w = __ldcs(reinterpret_cast<const uint4*>(g + m * ld + col0));
            const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k] += ew_to_float<T>(e[k]);
        }
    } else {
        for (long long m = m_begin + rgrp; m < m_end; m += BG_ROWS) {
#pragma unroll
            for (int k = 0; k < VEC; ++k)
                if (col0 + k < N) acc[k] += ew_to_float<T>(g[m * ld + col0 + k]);
        }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) part[rgrp][lane * VEC + k] = acc[k];
    __syncthreads();
    if (threadIdx.x < STRIP) {
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < BG_ROWS; ++r) s += part[r][threadIdx.x];
        strip_sum[threadIdx.x] = s;
    }
    // every CTA's strip_sum is complete and visible cluster-wide after this barrier
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (crank == 0 && threadIdx.x < STRIP) {
        const long long col = static_cast<long long>(blockIdx.x) * STRIP + threadIdx.x;
        float s = strip_sum[threadIdx.x];
        const uint32_t mine = static_cast<uint32_t>(__cvta_generic_to_shared(&strip_sum[threadIdx.x]));
        for (uint32_t r = 1; r < csize; ++r) {          // rank order: a fixed summation order
            uint32_t remote;
            float v;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(r));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
            s += v;
        }
        if (col < N) {
            if (out_f32 != nullptr) out_f32[col] = s;
            else out_t[col] = ew_from_float<T>(s);
        }
    }
    // no CTA may exit while CTA 0 still reads its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <typename T, int BG_LANES>
static cudaError_t bias_grad_lanes(const void* g, long long M, long long N, long long ld, void* out, int out_dtype, int csize,
                                   cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int STRIP = BG_LANES * VEC;
    const int vec = ((reinterpret_cast<uintptr_t>(g) & 15u) == 0 && (ld * sizeof(T)) % 16 == 0) ? 1 : 0;
    const long long strips = (N + STRIP - 1) / STRIP;
    if (strips > 0x7FFFFFFFll) return cudaErrorInvalidValue;
    float* of = out_dtype == SM120_DTYPE_FLOAT32 ? static_cast<float*>(out) : nullptr;
    T* ot = out_dtype == SM120_DTYPE_FLOAT32 ? nullptr : static_cast<T*>(out);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(strips), static_cast<unsigned>(csize), 1);
    cfg.blockDim = dim3(EW_THREADS, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = static_cast<unsigned>(csize);
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, sm120_bias_grad_kernel<T, BG_LANES>, static_cast<const T*>(g), M, N, ld, of, ot, vec);
}

template <typename T>
static cudaError_t bias_grad_typed(const void* g, long long M, long long N, long long ld, void* out, int out_dtype, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    // rows are split over a cluster when there are enough of them to give every CTA several steps of the widest strip
    int csize = 1;
    while (csize < BG_MAX_CLUSTER && M >= static_cast<long long>(csize) * 2 * 8 * 32) csize *= 2;
    // the widest strip that still gives the GPU enough CTAs
    const auto ctas = [&](int lanes) { return ((N + lanes * VEC - 1) / (lanes * VEC)) * csize; };
    if (ctas(32) >= BG_MIN_CTAS) return bias_grad_lanes<T, 32>(g, M, N, ld, out, out_dtype, csize, stream);
    if (ctas(16) >= BG_MIN_CTAS) return bias_grad_lanes<T, 16>(g, M, N, ld, out, out_dtype, csize, stream);
    return bias_grad_lanes<T, 8>(g, M, N, ld, out, out_dtype, csize, stream);
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
