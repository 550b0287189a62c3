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
// 256 threads as a 16 x 16 grid; CTA tile BMT x BNT (128x128, 128x64 or 64x64),
// K step 16; thread (ty, tx) owns rows ty*4 + 64*h + i and columns tx*4 + 64*g + j.
// Tiles of A and B are converted to fp32 and stored k-major in shared memory
// ([k][m], [k][n]) so the inner product reads them with 16-byte loads.  The next
// K step's global loads are issued into registers before the current step's
// FMAs (software pipelining); fp32 operands that are 16-byte aligned along their
// contiguous dimension are fetched with 16-byte loads.

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
    int vec_a, vec_b;          // fp32 operand may be read with 16-byte loads along its contiguous dimension
};

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_float<__nv_fp8_e4m3>(__nv_fp8_e4m3 v) { return float(v); }

constexpr int SIMT_BK = 16;
constexpr int SIMT_THREADS = 256;

// Global -> registers for one operand tile of ROWS (M or N) x 16 (K).  Element e of
// the thread's share is addressed so that consecutive threads walk the contiguous
// dimension of the stored matrix.  `k_contig`: K is the contiguous dimension.
template <typename T, int ROWS>
struct TileLoader {
    static constexpr int PER_THREAD = ROWS * SIMT_BK / SIMT_THREADS;   // 8 or 4
    float r[PER_THREAD];

    __device__ __forceinline__ void load(const T* X, long long ld, long long row0, long long k0, long long rows, long long K,
                                         bool k_contig, bool vec, int tid) {
        if (vec) {
            // 16-byte loads of fp32 (only instantiated meaningfully for T = float; `vec` is false otherwise)
            const float* Xf = reinterpret_cast<const float*>(X);
#pragma unroll
            for (int i = 0; i < PER_THREAD / 4; ++i) {
                const int q = tid + i * SIMT_THREADS;              // which float4
                long long row, k;
                if (k_contig) { k = k0 + (q % 4) * 4; row = row0 + q / 4; }
                else          { row = row0 + (q % (ROWS / 4)) * 4; k = k0 + q / (ROWS / 4); }
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (k_contig) {
                    if (row < rows && k + 3 < K) v = __ldg(reinterpret_cast<const float4*>(Xf + row * ld + k));
                    else if (row < rows) {
                        float t[4] = {0.f, 0.f, 0.f, 0.f};
                        for (int j = 0; j < 4; ++j) if (k + j < K) t[j] = Xf[row * ld + k + j];
                        v = make_float4(t[0], t[1], t[2], t[3]);
                    }
                } else {
                    if (k < K && row + 3 < rows) v = __ldg(reinterpret_cast<const float4*>(Xf + k * ld + row));
                    else if (k < K) {
                        float t[4] = {0.f, 0.f, 0.f, 0.f};
                        for (int j = 0; j < 4; ++j) if (row + j < rows) t[j] = Xf[k * ld + row + j];
                        v = make_float4(t[0], t[1], t[2], t[3]);
                    }
                }
                r[4 * i + 0] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < PER_THREAD; ++i) {
                const int e = tid + i * SIMT_THREADS;
                int row, k;
                if (k_contig) { k = e % SIMT_BK; row = e / SIMT_BK; } else { row = e % ROWS; k = e / ROWS; }
                const long long gr = row0 + row, gk = k0 + k;
                float v = 0.0f;
                if (gr < rows && gk < K) v = to_float<T>(k_contig ? X[gr * ld + gk] : X[gk * ld + gr]);
                r[i] = v;
            }
        }
    }

    // registers -> shared tile S[k][row]
    template <int PITCH>
    __device__ __forceinline__ void store(float (*S)[PITCH], bool k_contig, bool vec, int tid) const {
        if (vec) {
#pragma unroll
            for (int i = 0; i < PER_THREAD / 4; ++i) {
                const int q = tid + i * SIMT_THREADS;
                if (k_contig) {
                    const int k = (q % 4) * 4, row = q / 4;
#pragma unroll
                    for (int j = 0; j < 4; ++j) S[k + j][row] = r[4 * i + j];
                } else {
                    const int row = (q % (ROWS / 4)) * 4, k = q / (ROWS / 4);
                    *reinterpret_cast<float4*>(&S[k][row]) = make_float4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < PER_THREAD; ++i) {
                const int e = tid + i * SIMT_THREADS;
                int row, k;
                if (k_contig) { k = e % SIMT_BK; row = e / SIMT_BK; } else { row = e % ROWS; k = e / ROWS; }
                S[k][row] = r[i];
            }
        }
    }
};

template <typename T, int BMT, int BNT>
__global__ void __launch_bounds__(SIMT_THREADS)
sm120_gemm_simt_kernel(const SimtParams p) {
    constexpr int TM = BMT / 16, TN = BNT / 16;      // outputs per thread: 8 or 4 in each direction
    __shared__ __align__(16) float As[SIMT_BK][BMT + 4];
    __shared__ __align__(16) float Bs[SIMT_BK][BNT + 4];

    const int tid = threadIdx.x;
    const int tx = tid & 15;
    const int ty = tid >> 4;
    const long long bz = blockIdx.z;
    const long long m0 = static_cast<long long>(blockIdx.y) * BMT;
    const long long n0 = static_cast<long long>(blockIdx.x) * BNT;

    const T* A = static_cast<const T*>(p.A) + bz * p.stride_a;
    const T* B = static_cast<const T*>(p.B) + bz * p.stride_b;
    const bool a_kc = p.transpose_a == 0;     // A stored [M,K]: K contiguous
    const bool b_kc = p.transpose_b != 0;     // B stored [N,K]: K contiguous
    const bool a_vec = p.vec_a != 0, b_vec = p.vec_b != 0;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    TileLoader<T, BMT> la;
    TileLoader<T, BNT> lb;
    if (p.K > 0) {
        la.load(A, p.lda, m0, 0, p.M, p.K, a_kc, a_vec, tid);
        lb.load(B, p.ldb, n0, 0, p.N, p.K, b_kc, b_vec, tid);
    }
    for (long long k0 = 0; k0 < p.K; k0 += SIMT_BK) {
        la.template store<BMT + 4>(As, a_kc, a_vec, tid);
        lb.template store<BNT + 4>(Bs, b_kc, b_vec, tid);
        __syncthreads();
        if (k0 + SIMT_BK < p.K) {          // next K step's operands travel while this step is multiplied
            la.load(A, p.lda, m0, k0 + SIMT_BK, p.M, p.K, a_kc, a_vec, tid);
            lb.load(B, p.ldb, n0, k0 + SIMT_BK, p.N, p.K, b_kc, b_vec, tid);
        }
#pragma unroll
        for (int k = 0; k < SIMT_BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; i += 4) {
                const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4 + i * 16]);
                a[i] = av.x; a[i + 1] = av.y; a[i + 2] = av.z; a[i + 3] = av.w;
            }
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                const float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4 + j * 16]);
                b[j] = bv.x; b[j + 1] = bv.y; b[j + 2] = bv.z; b[j + 3] = bv.w;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

    float alpha = p.alpha;
    if (p.scale_a_dev != nullptr) alpha /= __ldg(p.scale_a_dev);
    if (p.scale_b_dev != nullptr) alpha /= __ldg(p.scale_b_dev);

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const long long gm = m0 + ty * 4 + (i / 4) * 64 + (i % 4);
        if (gm >= p.M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
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
static cudaError_t launch_typed(const GemmProblem& g, const SimtParams& sp, int shape, const char** name, const char* const names[3]) {
    auto grid_for = [&](int bm, int bn) {
        return dim3(static_cast<unsigned>((g.N + bn - 1) / bn), static_cast<unsigned>((g.M + bm - 1) / bm), static_cast<unsigned>(g.batch));
    };
    if (name) *name = names[shape];
    if (shape == 0)      sm120_gemm_simt_kernel<T, 128, 128><<<grid_for(128, 128), SIMT_THREADS, 0, g.stream>>>(sp);
    else if (shape == 1) sm120_gemm_simt_kernel<T, 128, 64><<<grid_for(128, 64), SIMT_THREADS, 0, g.stream>>>(sp);
    else                 sm120_gemm_simt_kernel<T, 64, 64><<<grid_for(64, 64), SIMT_THREADS, 0, g.stream>>>(sp);
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
    auto vec_ok = [&](const void* ptr, long long ld, long long stride) {
        return g.in_dtype == SM120_DTYPE_FLOAT32 && (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0 && ld % 4 == 0 && stride % 4 == 0;
    };
    sp.vec_a = vec_ok(g.A, g.lda, g.stride_a) ? 1 : 0;
    sp.vec_b = vec_ok(g.B, g.ldb, g.stride_b) ? 1 : 0;

    // grid.y and grid.z are limited to 65535
    if ((g.M + 63) / 64 > 65535 || g.batch > 65535) return cudaErrorInvalidValue;

    // the largest tile that still gives every SM work
    const long long t128 = ((g.M + 127) / 128) * ((g.N + 127) / 128) * g.batch;
    const long long t12864 = ((g.M + 127) / 128) * ((g.N + 63) / 64) * g.batch;
    const int shape = t128 >= 2ll * g.sm_count ? 0 : (5 * t12864 >= 4ll * g.sm_count ? 1 : 2);

    static const char* const f32[3] = {"simt_f32_128x128x16", "simt_f32_128x64x16", "simt_f32_64x64x16"};
    static const char* const f16[3] = {"simt_f16_128x128x16", "simt_f16_128x64x16", "simt_f16_64x64x16"};
    static const char* const b16[3] = {"simt_bf16_128x128x16", "simt_bf16_128x64x16", "simt_bf16_64x64x16"};
    static const char* const e4[3] = {"simt_e4m3_128x128x16", "simt_e4m3_128x64x16", "simt_e4m3_64x64x16"};
    switch (g.in_dtype) {
        case SM120_DTYPE_FLOAT32:  return launch_typed<float>(g, sp, shape, kernel_name, f32);
        case SM120_DTYPE_FLOAT16:  return launch_typed<__half>(g, sp, shape, kernel_name, f16);
        case SM120_DTYPE_BFLOAT16: return launch_typed<__nv_bfloat16>(g, sp, shape, kernel_name, b16);
        case SM120_DTYPE_FP8_E4M3: return launch_typed<__nv_fp8_e4m3>(g, sp, shape, kernel_name, e4);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace sm120
