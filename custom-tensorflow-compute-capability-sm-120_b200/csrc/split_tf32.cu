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
// contiguous in memory and X[k*ld + r] otherwise.
struct SplitJob {
    const float* X;
    float* X2;
    long long rows, ld, stride_x;
    int k_contiguous;
    unsigned row_tiles, batches;
};

// One 32 x 32 tile of op(X) per block, 32 x 8 threads; both operands in ONE launch (grid z: A's batch entries, then
// B's), because at the sizes where fp32 products are small the launches cost as much as the work.
__global__ void __launch_bounds__(256)
sm120_split_tf32_kernel(const SplitJob ja, const SplitJob jb, long long K, long long Kp) {
    // the GEMM that consumes the split operands may start its set-up now; it waits for this grid before it reads
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float tile[32][33];
    const bool is_a = blockIdx.z < ja.batches;
    const SplitJob& job = is_a ? ja : jb;
    if (blockIdx.y >= job.row_tiles) return;
    const long long bz = is_a ? blockIdx.z : blockIdx.z - ja.batches;
    const long long rows = job.rows, ld = job.ld;
    const int k_contiguous = job.k_contiguous;
    const float* x = job.X + bz * job.stride_x;
    float* x2 = job.X2 + bz * rows * 2 * Kp;
    const long long r0 = static_cast<long long>(blockIdx.y) * 32;
    const long long k0 = static_cast<long long>(blockIdx.x) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    // load op(X)[r0 + .., k0 + ..] into tile[r][k], walking the contiguous dimension with tx
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = ty + 8 * i;
        float v = 0.0f;
        if (k_contiguous) {
            const long long r = r0 + j, k = k0 + tx;
            if (r < rows && k < K) v = x[r * ld + k];
            tile[j][tx] = v;
        } else {
            const long long k = k0 + j, r = r0 + tx;
            if (r < rows && k < K) v = x[k * ld + r];
            tile[tx][j] = v;
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = ty + 8 * i;
        const long long r = r0 + j, k = k0 + tx;         // k < Kp always: the grid covers Kp / 32 tiles
        if (r >= rows) continue;
        const float v = tile[j][tx];
        const float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
        const float lo = __uint_as_float(__float_as_uint(v - hi) & 0xFFFFE000u);
        float* row = x2 + r * 2 * Kp;
        row[k] = hi;
        row[Kp + k] = lo;
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
    const SplitJob ja{static_cast<const float*>(p.A), a2, p.M, p.lda, p.stride_a, p.transpose_a ? 0 : 1,
                      static_cast<unsigned>((p.M + 31) / 32), static_cast<unsigned>(nb_a)};
    const SplitJob jb{static_cast<const float*>(p.B), b2, p.N, p.ldb, p.stride_b, p.transpose_b ? 1 : 0,
                      static_cast<unsigned>((p.N + 31) / 32), static_cast<unsigned>(nb_b)};
    const dim3 grid(static_cast<unsigned>(kp / 32), ja.row_tiles > jb.row_tiles ? ja.row_tiles : jb.row_tiles,
                    static_cast<unsigned>(nb_a + nb_b));
    sm120_split_tf32_kernel<<<grid, 256, 0, p.stream>>>(ja, jb, p.K, kp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;

    return tc_launch(g, wait_limit_ns, kernel_name);
}

}  // namespace sm120
