/*
 * Plain-C restatement of the reference's matmul semantics.  TEST INFRASTRUCTURE
 * ONLY: tests/ and bench.py's CPU-baseline legs load it; the product never does.
 * PARITY UNPINNED (see oracle/reference.py for why).
 *
 * One output element at a time, fp32 accumulator, ascending k, one fused
 * multiply-add per term:
 *   - accumulator and alpha/beta epilogue as sm120_matmul_kernel<T>
 *     (src/cuda_kernels/sm120_pure_kernels.cu:35,50-63): result = alpha*acc,
 *     C is read only when beta != 0;
 *   - transposes, pitches and strided batch as sm120_dynamic_matmul_kernel<T>
 *     (src/cuda_kernels/sm120_dynamic_shapes.cu:121-182), whose sm120_fma is
 *     __fmaf_rn (src/cuda_kernels/sm120_datatype_support.h:205-220).
 * Inputs are fp32 arrays holding the (already quantised) operand values; the
 * result is left in fp32 and the caller rounds it to the output type.
 */
#include <math.h>
#include <stdint.h>

int sm120_ref_matmul_f32(const float* A, const float* B, float* C,
                         int64_t M, int64_t N, int64_t K,
                         int64_t lda, int64_t ldb, int64_t ldc,
                         int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_c,
                         int transpose_a, int transpose_b, float alpha, float beta)
{
    if (M < 0 || N < 0 || K < 0 || batch < 1) return 1;
    for (int64_t bz = 0; bz < batch; ++bz) {
        const float* a = A + bz * stride_a;
        const float* b = B + bz * stride_b;
        float* c = C + bz * stride_c;
        for (int64_t i = 0; i < M; ++i) {
            for (int64_t j = 0; j < N; ++j) {
                float acc = 0.0f;
                for (int64_t k = 0; k < K; ++k) {
                    const float av = transpose_a ? a[k * lda + i] : a[i * lda + k];
                    const float bv = transpose_b ? b[j * ldb + k] : b[k * ldb + j];
                    acc = fmaf(av, bv, acc);
                }
                float r = alpha * acc;
                if (beta != 0.0f) r += beta * c[i * ldc + j];
                c[i * ldc + j] = r;
            }
        }
    }
    return 0;
}
