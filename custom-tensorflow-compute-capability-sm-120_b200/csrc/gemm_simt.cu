// SIMT (FFMA) GEMM for B200: the exact fp32 path of the SM120 matmul op and the
// path for operands that TMA cannot describe (unaligned pointers or pitches,
// K == 0).  Same contract as the tensor-core kernel: any input dtype, fp32
// accumulation in ascending k order per output element, transposes, pitches,
// strided batch, fused alpha/beta/bias/activation/cast epilogue.
//
// It replaces sm120_matmul_kernel<T> (src/cuda_kernels/sm120_pure_kernels.cu:19-65)
// and the fp32 tiled kernel of
// src/cuda_kernels/sm120_optimized_kernels_fixed.cu:46-101, and has the batch /
// transpose semantics of sm120_dynamic_matmul_kernel<T>
// (src/cuda_kernels/sm120_dynamic_shapes.cu:107-183).
//
// Two tile shapes: 128x128x16 with 8x8 outputs per thread for problems large
// enough to fill the GPU, 64x64x16 with 4x4 per thread otherwise.  256 threads.
// Tiles of A and B are converted to fp32 on the way into shared memory, stored
// k-major ([k][m], [k][n]) so the inner product reads them with 16-byte loads.

#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_common.h"

namespace sm120 {

struct SimtParams {
    const void* A;
    const void* B;
    void* C;
    const void* bias;
    long long M, N, K;
    long long lda, ldb, ldc;
    long long stride_a, stride_b, stride_c;
    int transpose_a, transpose_b;
    int out_dtype, bias_dtype;
    float alpha, beta;
    const float* scale_a_dev;
    const float* scale_b_dev;
    int activation;
};

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_float<__nv_fp8_e4m3>(__nv_fp8_e4m3 v) { return float(v); }

constexpr int SIMT_BK = 16;
constexpr int SIMT_THREADS = 256;

template <typename T, int TILE, int TT>   // TILE x TILE outputs per CTA, TT x TT per thread; TILE / TT == 16
__global__ void __launch_bounds__(SIMT_THREADS)
sm120_gemm_simt_kernel(const SimtParams p) {
    static_assert(TILE / TT == 16, "256 threads as a 16 x 16 grid");
    __shared__ __align__(16) float As[SIMT_BK][TILE + 4];
    __shared__ __align__(16) float Bs[SIMT_BK][TILE + 4];

    const int tid = threadIdx.x;
    const int tx = tid & 15;
    const int ty = tid >> 4;
    const long long bz = blockIdx.z;
    const long long m0 = static_cast<long long>(blockIdx.y) * TILE;
    const long long n0 = static_cast<long long>(blockIdx.x) * TILE;

    const T* A = static_cast<const T*>(p.A) + bz * p.stride_a;
    const T* B = static_cast<const T*>(p.B) + bz * p.stride_b;

    float acc[TT][TT];
#pragma unroll
    for (int i = 0; i < TT; ++i)
#pragma unroll
        for (int j = 0; j < TT; ++j) acc[i][j] = 0.0f;

    constexpr int PER_THREAD = TILE * SIMT_BK / SIMT_THREADS;

    for (long long k0 = 0; k0 < p.K; k0 += SIMT_BK) {
        // A tile -> As[k][m]; consecutive threads walk the contiguous dimension of the stored matrix
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int e = tid + i * SIMT_THREADS;
            int m, k;
            if (p.transpose_a) { m = e % TILE; k = e / TILE; } else { k = e % SIMT_BK; m = e / SIMT_BK; }
            const long long gm = m0 + m, gk = k0 + k;
            float v = 0.0f;
            if (gm < p.M && gk < p.K) v = to_float<T>(p.transpose_a ? A[gk * p.lda + gm] : A[gm * p.lda + gk]);
            As[k][m] = v;
        }
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int e = tid + i * SIMT_THREADS;
            int n, k;
            if (p.transpose_b) { k = e % SIMT_BK; n = e / SIMT_BK; } else { n = e % TILE; k = e / TILE; }
            const long long gn = n0 + n, gk = k0 + k;
            float v = 0.0f;
            if (gn < p.N && gk < p.K) v = to_float<T>(p.transpose_b ? B[gn * p.ldb + gk] : B[gk * p.ldb + gn]);
            Bs[k][n] = v;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < SIMT_BK; ++k) {
            float a[TT], b[TT];
#pragma unroll
            for (int i = 0; i < TT; i += 4) {
                const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4 + i * 16]);
                a[i] = av.x; a[i + 1] = av.y; a[i + 2] = av.z; a[i + 3] = av.w;
                const float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4 + i * 16]);
                b[i] = bv.x; b[i + 1] = bv.y; b[i + 2] = bv.z; b[i + 3] = bv.w;
            }
#pragma unroll
            for (int i = 0; i < TT; ++i)
#pragma unroll
                for (int j = 0; j < TT; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

    float alpha = p.alpha;
    if (p.scale_a_dev != nullptr) alpha /= __ldg(p.scale_a_dev);
    if (p.scale_b_dev != nullptr) alpha /= __ldg(p.scale_b_dev);

    // Thread (ty, tx) owns rows ty*4 + 64*(i/4) + i%4 and columns tx*4 + 64*(j/4) + j%4.
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        const long long gm = m0 + ty * 4 + (i / 4) * 64 + (i % 4);
        if (gm >= p.M) continue;
#pragma unroll
        for (int j = 0; j < TT; ++j) {
            const long long gn = n0 + tx * 4 + (j / 4) * 64 + (j % 4);
            if (gn >= p.N) continue;
            const long long off = bz * p.stride_c + gm * p.ldc + gn;
            float v = alpha * acc[i][j];
            if (p.beta != 0.0f) v += p.beta * load_as_float(p.C, off, p.out_dtype);
            if (p.bias != nullptr) v += load_as_float(p.bias, gn, p.bias_dtype);
            v = apply_activation(v, p.activation);
            store_from_float(p.C, off, p.out_dtype, v);
        }
    }
}

template <typename T>
static cudaError_t launch_typed(const GemmProblem& g, const SimtParams& sp, bool big, const char** name, const char* nbig,
                                const char* nsmall) {
    if (big) {
        dim3 grid(static_cast<unsigned>((g.N + 127) / 128), static_cast<unsigned>((g.M + 127) / 128), static_cast<unsigned>(g.batch));
        if (name) *name = nbig;
        sm120_gemm_simt_kernel<T, 128, 8><<<grid, SIMT_THREADS, 0, g.stream>>>(sp);
    } else {
        dim3 grid(static_cast<unsigned>((g.N + 63) / 64), static_cast<unsigned>((g.M + 63) / 64), static_cast<unsigned>(g.batch));
        if (name) *name = nsmall;
        sm120_gemm_simt_kernel<T, 64, 4><<<grid, SIMT_THREADS, 0, g.stream>>>(sp);
    }
    return cudaGetLastError();
}

cudaError_t simt_launch(const GemmProblem& g, const char** kernel_name) {
    SimtParams sp{};
    sp.A = g.A; sp.B = g.B; sp.C = g.C; sp.bias = g.bias;
    sp.M = g.M; sp.N = g.N; sp.K = g.K;
    sp.lda = g.lda; sp.ldb = g.ldb; sp.ldc = g.ldc;
    sp.stride_a = g.stride_a; sp.stride_b = g.stride_b; sp.stride_c = g.stride_c;
    sp.transpose_a = g.transpose_a; sp.transpose_b = g.transpose_b;
    sp.out_dtype = g.out_dtype; sp.bias_dtype = g.bias_dtype;
    sp.alpha = g.alpha * g.inv_scale; sp.beta = g.beta;
    sp.scale_a_dev = g.scale_a_dev; sp.scale_b_dev = g.scale_b_dev;
    sp.activation = g.activation;

    // grid.y and grid.z are limited to 65535
    if ((g.M + 63) / 64 > 65535 || g.batch > 65535) return cudaErrorInvalidValue;

    const long long tiles128 = ((g.M + 127) / 128) * ((g.N + 127) / 128) * g.batch;
    const bool big = tiles128 >= 2ll * g.sm_count;

    switch (g.in_dtype) {
        case SM120_DTYPE_FLOAT32:  return launch_typed<float>(g, sp, big, kernel_name, "simt_f32_128x128x16", "simt_f32_64x64x16");
        case SM120_DTYPE_FLOAT16:  return launch_typed<__half>(g, sp, big, kernel_name, "simt_f16_128x128x16", "simt_f16_64x64x16");
        case SM120_DTYPE_BFLOAT16: return launch_typed<__nv_bfloat16>(g, sp, big, kernel_name, "simt_bf16_128x128x16", "simt_bf16_64x64x16");
        case SM120_DTYPE_FP8_E4M3: return launch_typed<__nv_fp8_e4m3>(g, sp, big, kernel_name, "simt_e4m3_128x128x16", "simt_e4m3_64x64x16");
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace sm120
