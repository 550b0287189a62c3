// fp32 GEMM on the tensor cores by the 3xTF32 split.
//
// The tcgen05 tf32 MMA reads fp32 words and uses 10 mantissa bits.  Each fp32
// operand value x is split into  hi = x with its low 13 mantissa bits cleared
// and  lo = (x - hi) with its low 13 bits cleared  (x - hi is exact), both
// exactly representable in tf32.  Then
//     A.B  ~=  A_hi.B_hi + A_hi.B_lo + A_lo.B_hi          (lo.lo dropped: 2^-22 relative)
// is ONE tf32 GEMM whose k-blocks each issue three products.  The split kernel below writes
//     A2[m, :] = [ A_hi[m, :] | A_lo[m, :] ]     (K-major, pitch 2*Kp)
//     B2[n, :] = [ B_hi[:, n] | B_lo[:, n] ]     (K-major, pitch 2*Kp)
// with Kp = K rounded up to 32 and zero padding into caller-provided workspace, handling the
// caller's transposes and pitches, so the GEMM always sees two K-major operands; the GEMM kernel
// (the same as for the 16-bit types) loads the hi and lo tiles of both operands into one pipeline
// stage and accumulates the three products in fp32 in TMEM.  (A K dimension three times as long,
// [hi | hi | lo] . [hi | lo | hi], gives the same sums but fills shared memory 1.5x as often, and that
// fill, 96 bytes per clock and SM, was what bounded the first version.)  The tensor cores truncate when
// they add into the fp32 accumulator, so a sum left in TMEM over the whole of K
// drifts by about K * 2^-27 relative (1.16e-5 measured at K = 1024, outside the
// op's 1e-5 gate); the GEMM therefore runs K in runs of six k-blocks, each into a
// zeroed accumulator, and the epilogue warps add the runs in registers with
// round-to-nearest (gemm_tcgen05_kernel.cuh), which keeps the error below 5e-6 at any K.
//
// This is the tensor-core answer to the reference's fp32 kernels
// (src/cuda_kernels/sm120_optimized_kernels_fixed.cu:46-101,
// src/cuda_kernels/sm120_pure_kernels.cu:19-65); the FFMA kernel in gemm_simt.cu
// remains the path when no workspace is given.

#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_common.h"

namespace sm120 {

// One operand's split: `rows` is M (for A) or N (for B); element (r, k) of op(X) is X[r*ld + k] when k is
// contiguous in memory and X[k*ld + r] otherwise.  `vec`: base, pitch and batch stride are multiples of 16 bytes and
// the contiguous extent is a multiple of 4 elements, so the operand can be read in 16-byte pieces.
struct SplitJob {
    const float* X;
    float* X2;
    long long rows, ld, stride_x;
    int k_contiguous, vec;
    unsigned row_tiles, batches;
};

constexpr int SPLIT_TILE = 64;           // rows and K elements of op(X) per block

__device__ __forceinline__ void split_hi_lo(float v, float& hi, float& lo) {
    hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    lo = __uint_as_float(__float_as_uint(v - hi) & 0xFFFFE000u);
}

__device__ __forceinline__ void split_store4(float* row, long long k, long long Kp, const float4 v) {
    float4 hi, lo;
    split_hi_lo(v.x, hi.x, lo.x);
    split_hi_lo(v.y, hi.y, lo.y);
    split_hi_lo(v.z, hi.z, lo.z);
    split_hi_lo(v.w, hi.w, lo.w);
    *reinterpret_cast<float4*>(row + k) = hi;
    *reinterpret_cast<float4*>(row + Kp + k) = lo;
}

// One 64 x 64 tile of op(X) per block of 256 threads; both operands in ONE launch (grid z: A's batch entries, then
// B's), because at the sizes where fp32 products are small the launches cost as much as the work.  The pass is
// HBM-bound (4 bytes read, 8 written per element): aligned operands move in 16-byte pieces, 256 contiguous bytes per
// row and 16 threads, directly when K is the contiguous dimension and through a shared-memory transpose when it is
// not; anything else takes the element-wise path.
__global__ void __launch_bounds__(256)
sm120_split_tf32_kernel(const SplitJob ja, const SplitJob jb, long long K, long long Kp) {
    // the GEMM that consumes the split operands may start its set-up now; it waits for this grid before it reads
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float tile[SPLIT_TILE][SPLIT_TILE + 1];
    const bool is_a = blockIdx.z < ja.batches;
    const SplitJob& job = is_a ? ja : jb;
    if (blockIdx.y >= job.row_tiles) return;
    const long long bz = is_a ? blockIdx.z : blockIdx.z - ja.batches;
    const long long rows = job.rows, ld = job.ld;
    const int k_contiguous = job.k_contiguous;
    const float* x = job.X + bz * job.stride_x;
    float* x2 = job.X2 + bz * rows * 2 * Kp;
    const long long r0 = static_cast<long long>(blockIdx.y) * SPLIT_TILE;
    const long long k0 = static_cast<long long>(blockIdx.x) * SPLIT_TILE;
    if (job.vec) {
        const int l16 = threadIdx.x & 15, sub = threadIdx.x >> 4;     // 16 threads x 16 bytes per row piece, 16 pieces per step
        if (k_contiguous) {
            const long long k = k0 + l16 * 4;                         // K % 4 == 0: a piece is inside K or outside
            if (k >= Kp) return;
            float4 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const long long r = r0 + sub + 16 * i;
                v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (r < rows && k < K) v[i] = __ldcs(reinterpret_cast<const float4*>(x + r * ld + k));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const long long r = r0 + sub + 16 * i;
                if (r < rows) split_store4(x2 + r * 2 * Kp, k, Kp, v[i]);
            }
            return;
        }
        // rows are the contiguous dimension (rows % 4 == 0): 16-byte pieces along r in, a transpose, 16-byte pieces along k out
        {
            const long long r = r0 + l16 * 4;
            float4 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const long long k = k0 + sub + 16 * i;
                v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (k < K && r < rows) v[i] = __ldcs(reinterpret_cast<const float4*>(x + k * ld + r));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int kk = sub + 16 * i;
                tile[kk][l16 * 4 + 0] = v[i].x;
                tile[kk][l16 * 4 + 1] = v[i].y;
                tile[kk][l16 * 4 + 2] = v[i].z;
                tile[kk][l16 * 4 + 3] = v[i].w;
            }
        }
        __syncthreads();
        const long long k = k0 + l16 * 4;
        if (k >= Kp) return;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rr = sub + 16 * i;
            const long long r = r0 + rr;
            if (r >= rows) continue;
            const float4 v = make_float4(tile[l16 * 4 + 0][rr], tile[l16 * 4 + 1][rr], tile[l16 * 4 + 2][rr], tile[l16 * 4 + 3][rr]);
            split_store4(x2 + r * 2 * Kp, k, Kp, v);
        }
        return;
    }
    // element-wise: four 32 x 32 sub-tiles, walking the contiguous dimension with tx
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll 1
    for (int q = 0; q < 4; ++q) {
        const long long rq = r0 + 32 * (q >> 1), kq = k0 + 32 * (q & 1);
        if (q != 0) __syncthreads();                                  // the previous sub-tile has been read
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = ty + 8 * i;
            float v = 0.0f;
            if (k_contiguous) {
                const long long r = rq + j, k = kq + tx;
                if (r < rows && k < K) v = x[r * ld + k];
                tile[j][tx] = v;
            } else {
                const long long k = kq + j, r = rq + tx;
                if (r < rows && k < K) v = x[k * ld + r];
                tile[tx][j] = v;
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = ty + 8 * i;
            const long long r = rq + j, k = kq + tx;
            if (r >= rows || k >= Kp) continue;
            float hi, lo;
            split_hi_lo(tile[j][tx], hi, lo);
            float* row = x2 + r * 2 * Kp;
            row[k] = hi;
            row[Kp + k] = lo;
        }
    }
}

static long long padded_k(long long K) { return (K + 31) / 32 * 32; }

size_t tf32x3_workspace_bytes(const GemmProblem& p) {
    const long long kp = padded_k(p.K);
    const long long nb_b = (p.batch > 1 && p.stride_b == 0) ? 1 : p.batch;     // a broadcast B is split once
    const long long nb_a = (p.batch > 1 && p.stride_a == 0) ? 1 : p.batch;
    return static_cast<size_t>((p.M * nb_a + p.N * nb_b) * 2 * kp) * sizeof(float);
}

cudaError_t tf32x3_launch(const GemmProblem& p, void* workspace, uint64_t wait_limit_ns, const char** kernel_name) {
    const long long kp = padded_k(p.K);
    const long long nb_a = (p.batch > 1 && p.stride_a == 0) ? 1 : p.batch;
    const long long nb_b = (p.batch > 1 && p.stride_b == 0) ? 1 : p.batch;
    if (nb_a + nb_b > 65535 || (p.M + 31) / 32 > 65535 || (p.N + 31) / 32 > 65535) return cudaErrorInvalidValue;
    float* a2 = static_cast<float*>(workspace);
    float* b2 = a2 + p.M * nb_a * 2 * kp;
    // the GEMM over the split operands; checked before anything is enqueued, so a rejected call launches nothing
    GemmProblem g = p;
    g.A = a2; g.B = b2;
    g.K = 2 * kp;                       // [hi | lo]: the GEMM walks kp and reads both halves of a row per k-block
    g.lda = 2 * kp; g.ldb = 2 * kp;
    g.transpose_a = 0; g.transpose_b = 1;
    g.stride_a = (nb_a > 1) ? p.M * 2 * kp : 0;
    g.stride_b = (nb_b > 1) ? p.N * 2 * kp : 0;
    g.tf32_operands = 1;
    const char* why = nullptr;
    if (!tc_supported(g, &why)) return cudaErrorInvalidValue;
    // A: op(A)[m,k]; k is contiguous unless A is stored transposed.  B: op(B)^T[n,k]; k is contiguous when B is stored [N,K].
    const auto vec_ok = [&](const void* x, long long ld, long long stride, long long contiguous_extent) {
        return (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && ld % 4 == 0 && stride % 4 == 0 && contiguous_extent % 4 == 0 ? 1 : 0;
    };
    const int ka = p.transpose_a ? 0 : 1, kb = p.transpose_b ? 1 : 0;
    const SplitJob ja{static_cast<const float*>(p.A), a2, p.M, p.lda, p.stride_a, ka, vec_ok(p.A, p.lda, p.stride_a, ka ? p.K : p.M),
                      static_cast<unsigned>((p.M + SPLIT_TILE - 1) / SPLIT_TILE), static_cast<unsigned>(nb_a)};
    const SplitJob jb{static_cast<const float*>(p.B), b2, p.N, p.ldb, p.stride_b, kb, vec_ok(p.B, p.ldb, p.stride_b, kb ? p.K : p.N),
                      static_cast<unsigned>((p.N + SPLIT_TILE - 1) / SPLIT_TILE), static_cast<unsigned>(nb_b)};
    const dim3 grid(static_cast<unsigned>((kp + SPLIT_TILE - 1) / SPLIT_TILE), ja.row_tiles > jb.row_tiles ? ja.row_tiles : jb.row_tiles,
                    static_cast<unsigned>(nb_a + nb_b));
    sm120_split_tf32_kernel<<<grid, 256, 0, p.stream>>>(ja, jb, p.K, kp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;

    return tc_launch(g, wait_limit_ns, kernel_name);
}

}  // namespace sm120
