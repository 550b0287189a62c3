// Internal declarations shared by the launcher and the two kernel families of
// the SM120 matmul op for B200.  Nothing here is part of the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "../../include/sm120_c_interface.h"

namespace sm120 {

// A validated, fully resolved GEMM problem: what SM120GemmDesc says after the
// launcher has filled in tight pitches and checked every field.
struct GemmProblem {
    const void* A;
    const void* B;
    void* C;
    const void* bias;
    int64_t M, N, K;
    int64_t lda, ldb, ldc;           // elements
    int64_t batch;
    int64_t stride_a, stride_b, stride_c;  // elements
    int transpose_a, transpose_b;
    int in_dtype, out_dtype, bias_dtype;
    int tf32_operands;               // in_dtype FLOAT32 whose values already fit tf32 (low 13 mantissa bits zero)
    float alpha, beta;
    float inv_scale;                 // 1 / (scale_a * scale_b) from the by-value scales
    const float* scale_a_dev;
    const float* scale_b_dev;
    int activation;
    int optimization_level;
    cudaStream_t stream;
    int device;
    int sm_count;
    // further buffers that receive a copy of the [M, N] result (same pitch, batch stride and dtype as C):
    // other GPUs' memory when the launch also does the all-gather of an M-sharded product
    void* extra_dests[7];
    int num_extra_dests;
    int tuning;                      // SM120GemmDesc::tuning (SM120_TUNE_* bits)
    int64_t split_k;                 // 0, or: the `batch` entries are consecutive K ranges of this length of ONE product
                                     // (A and B are not batched; entry z writes its partial sums to C + z * stride_c)
    void* trace;                     // null, or the caller's buffer for SM120_TUNE_TRACE
};

__host__ __device__ inline int dtype_size(int dtype) {
    switch (dtype) {
        case SM120_DTYPE_FLOAT32: return 4;
        case SM120_DTYPE_FLOAT16: return 2;
        case SM120_DTYPE_BFLOAT16: return 2;
        case SM120_DTYPE_FP8_E4M3: return 1;
        default: return 0;
    }
}

// Can this problem be described to TMA and run on the tcgen05 kernel?
bool tc_supported(const GemmProblem& p, const char** why);

// Enqueue on p.stream.  Both return the launch status.
cudaError_t tc_launch(const GemmProblem& p, uint64_t wait_limit_ns, const char** kernel_name);
cudaError_t simt_launch(const GemmProblem& p, const char** kernel_name);

// fp32 on tensor cores (3xTF32): bytes of workspace the split operands need, and the launch
// (split kernels + tcgen05 kind::tf32 GEMM over the three partial products).
size_t tf32x3_workspace_bytes(const GemmProblem& p);
cudaError_t tf32x3_launch(const GemmProblem& p, void* workspace, uint64_t wait_limit_ns, const char** kernel_name);

// Split-K for products with too few output tiles to fill the GPU: the K range is cut into `splitk_factor` parts
// that run as the batch entries of one tcgen05 launch into fp32 workspace, and a second kernel adds the parts
// in a fixed order and applies alpha, beta, bias, activation and the output type.  splitk_factor returns 1 when
// the product should not be split (enough tiles, short K, batched, fp32, extra destinations, or switched off).
int splitk_factor(const GemmProblem& p);
size_t splitk_workspace_bytes(const GemmProblem& p);
cudaError_t splitk_launch(const GemmProblem& p, void* workspace, uint64_t wait_limit_ns, const char** kernel_name);

// Per-device status word of the tcgen05 kernel (0 = no wait ran out).
cudaError_t tc_read_status(unsigned int* status, int clear);
// SM cycles and nanoseconds that CTA 0 of the last tcgen05 launch on the current device was alive.
cudaError_t tc_read_probe(unsigned long long* cycles_ns);
// How many tensor maps this process has encoded / taken from a thread's cache so far.
void tc_map_cache_stats(uint64_t* encodes, uint64_t* hits);

// ---------------------------------------------------------------------------
// Epilogue math, shared by both kernel families.  Formulas and constants follow
// the reference's activation table (src/cuda_kernels/sm120_pure_kernels.cu:141-171);
// GELU_ERF is the exact GELU of the Keras path.  Compiled without fast-math.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float apply_activation(float x, int act) {
    switch (act) {
        case SM120_ACTIVATION_RELU:       return fmaxf(0.0f, x);
        case SM120_ACTIVATION_LEAKY_RELU: return x > 0.0f ? x : 0.01f * x;
        case SM120_ACTIVATION_ELU:        return x > 0.0f ? x : (expf(x) - 1.0f);
        case SM120_ACTIVATION_SELU:       return x > 0.0f ? 1.0507f * x : 1.0507f * 1.67326f * (expf(x) - 1.0f);
        case SM120_ACTIVATION_GELU:       return 0.5f * x * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x)));
        case SM120_ACTIVATION_SWISH:      return x / (1.0f + expf(-x));
        case SM120_ACTIVATION_MISH:       return x * tanhf(logf(1.0f + expf(x)));
        case SM120_ACTIVATION_TANH:       return tanhf(x);
        case SM120_ACTIVATION_SIGMOID:    return 1.0f / (1.0f + expf(-x));
        case SM120_ACTIVATION_GELU_ERF:   return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
        default:                          return x;
    }
}

__device__ __forceinline__ float load_as_float(const void* p, int64_t i, int dtype) {
    switch (dtype) {
        case SM120_DTYPE_FLOAT32:  return static_cast<const float*>(p)[i];
        case SM120_DTYPE_FLOAT16:  return __half2float(static_cast<const __half*>(p)[i]);
        case SM120_DTYPE_BFLOAT16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
        case SM120_DTYPE_FP8_E4M3: return float(static_cast<const __nv_fp8_e4m3*>(p)[i]);
        default: return 0.0f;
    }
}

__device__ __forceinline__ void store_from_float(void* p, int64_t i, int dtype, float v) {
    switch (dtype) {
        case SM120_DTYPE_FLOAT32:  static_cast<float*>(p)[i] = v; break;
        case SM120_DTYPE_FLOAT16:  static_cast<__half*>(p)[i] = __float2half_rn(v); break;
        case SM120_DTYPE_BFLOAT16: static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); break;
        default: break;
    }
}

}  // namespace sm120
