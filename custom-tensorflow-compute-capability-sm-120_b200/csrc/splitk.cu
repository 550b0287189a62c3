// Split-K for the tensor-core GEMM.
//
// A product with few output tiles and a long K (a [1024, 8192] x [8192, 1024] projection, a
// weight gradient, a decode-time [128, 4096] x [4096, 4096]) leaves most of the 148 SMs idle
// when every tile walks the whole of K on one CTA (pair).  Here the K range is cut into S
// consecutive parts that run as the S batch entries of ONE launch of the same tcgen05 kernel
// (entry z reads K coordinates [z K/S, (z + 1) K/S) of the unbatched operands and writes
// fp32 partial sums to workspace + z M N), and a second, HBM-bound kernel adds the S parts in
// ascending z - a fixed order, so the result is reproducible - and applies alpha, beta,
// bias, activation and the output type.  No atomics.  The reference has no counterpart: its
// kernels give one thread block per output tile whatever the shape
// (src/cuda_kernels/sm120_optimized_kernels_fixed.cu:46-101).

#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_common.h"

namespace sm120 {

namespace {

constexpr int SPLITK_MAX = 8;
constexpr int RED_THREADS = 256;

// out[m, n] = act(alpha * sum_z part[z][m][n] + beta * C[m, n] + bias[n]); 4 columns per thread where N allows
__global__ void __launch_bounds__(RED_THREADS)
sm120_splitk_reduce_kernel(const float* __restrict__ part, int splits, long long M, long long N, void* __restrict__ C, long long ldc,
                           int out_dtype, float alpha, float beta, const void* __restrict__ bias, int bias_dtype, int activation,
                           int vec) {
    // launched as a programmatic dependent of the GEMM: the blocks may be resident before the GEMM has finished, and
    // wait here until its partial sums are complete and visible
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long plane = M * N;
    if (vec) {
        const long long nv = N >> 2;
        const long long total = M * nv;
        for (long long i = static_cast<long long>(blockIdx.x) * RED_THREADS + threadIdx.x; i < total;
             i += static_cast<long long>(gridDim.x) * RED_THREADS) {
            const long long m = i / nv, n = (i - m * nv) << 2;
            const float4* src = reinterpret_cast<const float4*>(part + m * N + n);
            float4 s = __ldcs(src);
            for (int z = 1; z < splits; ++z) {
                const float4 v = __ldcs(reinterpret_cast<const float4*>(part + z * plane + m * N + n));
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            float r[4] = {s.x, s.y, s.z, s.w};
            const long long off = m * ldc + n;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float x = alpha * r[k];
                if (beta != 0.0f) x = fmaf(beta, load_as_float(C, off + k, out_dtype), x);
                if (bias != nullptr) x += load_as_float(bias, n + k, bias_dtype);
                r[k] = apply_activation(x, activation);
            }
            if (out_dtype == SM120_DTYPE_FLOAT32) {
                *reinterpret_cast<float4*>(static_cast<float*>(C) + off) = make_float4(r[0], r[1], r[2], r[3]);
            } else if (out_dtype == SM120_DTYPE_FLOAT16) {
                const __half2 a = __floats2half2_rn(r[0], r[1]), b = __floats2half2_rn(r[2], r[3]);
                *reinterpret_cast<uint2*>(static_cast<__half*>(C) + off) =
                    make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
            } else {
                const __nv_bfloat162 a = __floats2bfloat162_rn(r[0], r[1]), b = __floats2bfloat162_rn(r[2], r[3]);
                *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(C) + off) =
                    make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
            }
        }
    } else {
        for (long long i = static_cast<long long>(blockIdx.x) * RED_THREADS + threadIdx.x; i < plane;
             i += static_cast<long long>(gridDim.x) * RED_THREADS) {
            const long long m = i / N, n = i - m * N;
            float s = part[i];
            for (int z = 1; z < splits; ++z) s += part[z * plane + i];
            float x = alpha * s;
            const long long off = m * ldc + n;
            if (beta != 0.0f) x = fmaf(beta, load_as_float(C, off, out_dtype), x);
            if (bias != nullptr) x += load_as_float(bias, n, bias_dtype);
            store_from_float(C, off, out_dtype, apply_activation(x, activation));
        }
    }
}

}  // namespace

int splitk_factor(const GemmProblem& p) {
    if (p.tuning & SM120_TUNE_NO_SPLIT_K) return 1;
    if (p.in_dtype != SM120_DTYPE_FLOAT16 && p.in_dtype != SM120_DTYPE_BFLOAT16 && p.in_dtype != SM120_DTYPE_FP8_E4M3) return 1;
    if (p.batch != 1 || p.num_extra_dests != 0 || p.trace != nullptr || p.split_k != 0) return 1;
    if (p.M < 1 || p.N < 1 || p.sm_count < 1) return 1;
    const int64_t bk = 128 / dtype_size(p.in_dtype);             // elements of K per k-block
    if (p.K < 16 * bk) return 1;
    // output tiles of the shape the kernel takes when the tiles do not fill the GPU: 256 x 256 pairs when there are more
    // than 128 rows, else 128 x 128; the parts are chosen so that parts x tiles stays within one wave
    const bool pair = p.M > 128;
    const int64_t tiles = pair ? ((p.M + 255) / 256) * ((p.N + 255) / 256) : (p.N + 127) / 128;
    const int64_t slots = pair ? p.sm_count / 2 : p.sm_count;
    int64_t s = slots / tiles;
    if (s > SPLITK_MAX) s = SPLITK_MAX;
    // every part a whole number of k-blocks, at least eight of them
    while (s >= 2 && (p.K % (s * bk) != 0 || p.K / s < 8 * bk)) --s;
    return s >= 2 ? static_cast<int>(s) : 1;
}

size_t splitk_workspace_bytes(const GemmProblem& p) {
    const int s = splitk_factor(p);
    return s >= 2 ? static_cast<size_t>(s) * static_cast<size_t>(p.M) * static_cast<size_t>(p.N) * sizeof(float) : 0;
}

cudaError_t splitk_launch(const GemmProblem& p, void* workspace, uint64_t wait_limit_ns, const char** kernel_name) {
    const int s = splitk_factor(p);
    if (s < 2 || workspace == nullptr) return cudaErrorInvalidValue;
    GemmProblem g = p;
    g.batch = s;
    g.split_k = p.K / s;
    g.stride_a = 0; g.stride_b = 0;
    g.C = workspace; g.ldc = p.N; g.stride_c = p.M * p.N;
    g.out_dtype = SM120_DTYPE_FLOAT32;
    g.alpha = 1.0f; g.beta = 0.0f;           // the operand scales (by value and on the device) stay: they are linear
    g.bias = nullptr;
    g.activation = SM120_ACTIVATION_NONE;
    const char* why = nullptr;
    if (!tc_supported(g, &why)) return cudaErrorInvalidValue;
    cudaError_t e = tc_launch(g, wait_limit_ns, kernel_name);
    if (e != cudaSuccess) return e;
    const int out_es = dtype_size(p.out_dtype);
    const int vec = (p.N % 4 == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15u) == 0 && (p.ldc * out_es) % 16 == 0 &&
                     (p.out_dtype == SM120_DTYPE_FLOAT32 || (p.ldc * out_es) % 8 == 0)) ? 1 : 0;
    const long long work = vec ? p.M * (p.N / 4) : p.M * p.N;
    long long blocks = (work + RED_THREADS - 1) / RED_THREADS;
    const long long cap = static_cast<long long>(p.sm_count) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
    cfg.blockDim = dim3(RED_THREADS, 1, 1);
    cfg.stream = p.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // see griddepcontrol.wait in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, sm120_splitk_reduce_kernel, static_cast<const float*>(workspace), s,
                              static_cast<long long>(p.M), static_cast<long long>(p.N), p.C, static_cast<long long>(p.ldc), p.out_dtype,
                              p.alpha, p.beta, p.bias, p.bias_dtype, p.activation, vec);
}

}  // namespace sm120
