/*
 * C ABI of the B200 (sm_100a) build of the SM120 mixed-precision matmul op.
 *
 * This is the drop-in boundary: the entry points below are what the
 * TensorFlow OpKernel (SM120MatMulOp<T>::Compute) and any other foreign
 * caller (ctypes, cgo, JNI ...) bind.  Every signature uses plain pointers and
 * sizes; no C++ or framework type crosses it.  The library is built as
 * `_sm120_ops.so`, the artefact name the reference loads
 * (python/sm120_ops.py:29-31).
 *
 * Contract shared by every launcher here (same as the reference launcher,
 * src/cuda_kernels/sm120_c_interface.cu:32-60):
 *   - all matrix pointers are DEVICE pointers owned by the caller;
 *   - the launcher never allocates, frees or synchronises; work is enqueued on
 *     the caller's stream (0 = the default stream);
 *   - the return value is a cudaError_t: cudaSuccess when the kernel was
 *     enqueued, cudaErrorInvalidValue for a rejected argument (nothing is
 *     launched), otherwise the launch error;
 *   - the launchers are re-entrant and may be called from several host threads
 *     and for several devices at once.
 *   - there is no CPU fallback: on a device that is not compute capability
 *     10.x the launchers return cudaErrorInvalidDevice.
 */
#ifndef SM120_C_INTERFACE_H
#define SM120_C_INTERFACE_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Activation codes 0..8 keep the reference's numbering
 * (src/cuda_kernels/sm120_c_interface.h:21-31) and formulas
 * (src/cuda_kernels/sm120_pure_kernels.cu:141-171; code 4 is the tanh GELU
 * with constants 0.7978845608 / 0.044715).  Two codes are appended for the
 * fused GEMM epilogue: NONE (identity) and GELU_ERF, the exact erf GELU that
 * the Keras path computes (python/sm120_keras_layers.py:105,172). */
typedef enum {
    SM120_ACTIVATION_NONE = -1,
    SM120_ACTIVATION_RELU = 0,
    SM120_ACTIVATION_LEAKY_RELU = 1,
    SM120_ACTIVATION_ELU = 2,
    SM120_ACTIVATION_SELU = 3,
    SM120_ACTIVATION_GELU = 4,
    SM120_ACTIVATION_SWISH = 5,
    SM120_ACTIVATION_MISH = 6,
    SM120_ACTIVATION_TANH = 7,
    SM120_ACTIVATION_SIGMOID = 8,
    SM120_ACTIVATION_GELU_ERF = 9
} SM120ActivationType;

/* Values 0 and 1 are the reference's (src/cuda_kernels/sm120_c_interface.h:40-43).
 * BFLOAT16 and FP8_E4M3 are types the reference declares
 * (src/cuda_kernels/sm120_datatype_support.h:49-58,71-82) but never feeds to a
 * GEMM; they are appended here.  FP8_E4M3 is an input type only. */
typedef enum {
    SM120_DTYPE_FLOAT32 = 0,
    SM120_DTYPE_FLOAT16 = 1,
    SM120_DTYPE_BFLOAT16 = 2,
    SM120_DTYPE_FP8_E4M3 = 3
} SM120DataType;

/* Which kernel family a launch may use.  AUTO picks the tcgen05 tensor-core
 * kernel whenever the operands satisfy TMA's alignment rules and otherwise the
 * SIMT kernel; the other two values force one family (a forced tensor-core
 * launch of operands that cannot be described to TMA is rejected). */
typedef enum {
    SM120_PATH_AUTO = 0,
    SM120_PATH_TENSOR_CORE = 1,
    SM120_PATH_SIMT = 2
} SM120KernelPath;

/*
 * Replaces sm120_launch_matmul (src/cuda_kernels/sm120_c_interface.h:53-58,
 * body src/cuda_kernels/sm120_c_interface.cu:32-60) with the same signature:
 * C[M,N] = alpha * A[M,K] * B[K,N] + beta * C, all three row-major and dense,
 * inputs and output of type `dtype`, fp32 accumulation, C read only when
 * beta != 0 (src/cuda_kernels/sm120_pure_kernels.cu:58-63).
 * dtype FLOAT32 runs the exact FFMA kernel (this signature carries no
 * workspace for the tensor-core route); FLOAT16 / BFLOAT16 run the tcgen05
 * kernel.  An unknown dtype returns cudaErrorInvalidValue as the reference does.
 */
cudaError_t sm120_launch_matmul(
    const void* A, const void* B, void* C,
    int M, int N, int K,
    float alpha, float beta,
    SM120DataType dtype,
    cudaStream_t stream);

/*
 * Replaces launch_sm120_matmul
 * (src/cuda_kernels/sm120_optimized_kernels_fixed.cu:788-798): fp32
 * C[M,N] = A[M,K] * B[K,N], row-major.  Returns nothing, as the reference's
 * does; a failure is left in cudaGetLastError().
 */
void launch_sm120_matmul(
    const float* A, const float* B, float* C,
    int M, int N, int K,
    cudaStream_t stream);

/*
 * Superset descriptor.  It carries what the three competing OpKernel bodies
 * pass or need (transposes: src/tensorflow_ops/sm120_ops_fixed.cc:137-143;
 * alpha/beta: src/tensorflow_ops/sm120_tensorflow_ops.cc:93), the strided-batch
 * form of LaunchSM120DynamicMatMul
 * (src/cuda_kernels/sm120_dynamic_shapes.cu:107-183,323-383), and the fused
 * Dense epilogue (bias add + activation + cast) that the reference runs as
 * separate ops (python/sm120_keras_layers.py:159-174).
 *
 *   C[b] = act( alpha * inv_scale * op(A[b]) * op(B[b]) + beta * C[b] + bias )
 *
 * op(A) is [M,K]: A is stored row-major [M,K] with row pitch lda, or, when
 * transpose_a != 0, as [K,M].  op(B) is [K,N]: B is stored [K,N] with pitch
 * ldb, or [N,K] when transpose_b != 0.  C is [M,N] with pitch ldc.  A pitch of
 * 0 means "tight" (the stored row length).  Pitches and batch strides are in
 * elements.  inv_scale = 1 / (scale_a * scale_b): the per-tensor quantisation
 * scales of FP8 inputs (q = saturate_e4m3(x * scale)); both default to 1 when
 * given as 0.  When scale_a_dev / scale_b_dev are non-null they are device
 * pointers to one float each and override the by-value scales, so a producer
 * kernel can write them without a host round trip.
 * bias has N entries of bias_dtype (FLOAT32, FLOAT16 or BFLOAT16) or is null.
 */
typedef struct SM120GemmDesc {
    uint32_t struct_size;      /* sizeof(SM120GemmDesc); checked */
    int32_t  in_dtype;         /* SM120DataType of A and B */
    int32_t  out_dtype;        /* SM120DataType of C; FP8 is rejected */
    int32_t  bias_dtype;       /* SM120DataType of bias (ignored when bias is null) */
    const void* A;
    const void* B;
    void*       C;
    const void* bias;
    int64_t M, N, K;
    int64_t lda, ldb, ldc;
    int64_t batch;             /* >= 1 */
    int64_t stride_a, stride_b, stride_c;   /* elements between batch entries; 0 with batch > 1 broadcasts A or B */
    int32_t transpose_a, transpose_b;
    float   alpha, beta;
    float   scale_a, scale_b;
    const float* scale_a_dev;
    const float* scale_b_dev;
    int32_t activation;        /* SM120ActivationType */
    int32_t path;              /* SM120KernelPath */
    int32_t optimization_level;/* 0..2 as SM120Config.optimization_level (python/sm120_ops.py:108-122); 0 = conservative tile, 1/2 = tuned */
    int32_t tuning;            /* SM120_TUNE_* bits, 0 = every choice is the launcher's (see below) */
    cudaStream_t stream;
    void*    workspace;        /* optional device scratch owned by the caller (16-byte aligned), or null */
    uint64_t workspace_bytes;  /* its size; see sm120_matmul_workspace_bytes and SM120_TUNE_TRACE */
} SM120GemmDesc;

/*
 * Per-call overrides of the tensor-core launcher's own choices, for tests and
 * tuning runs.  They live in the descriptor, not in the library, so one thread's
 * experiment never changes another thread's launch.  0 asks for nothing.  An
 * override that the chosen kernel has no variant for is ignored.
 *   CTA_GROUP_1 / _2     single-CTA tiles (128 x BN) / CTA-pair tiles (256 x 256)
 *   EPI_WARPS_8 / _16    epilogue warps per CTA (16 exists for pair tiles only)
 *   NO_SPLIT_TAIL        a short last wave is not cut into half-width tiles
 *   NO_SPLIT_K           the K range is never cut into parts (see sm120_matmul_workspace_bytes)
 *   GROUP_M(g)           raster group of g row tiles, 1 <= g <= 255 (0 = heuristic)
 *   STALL_KBLOCK(kb)     self-test of the bounded waits: every TMA producer stops
 *                        before k-block kb (0 <= kb <= 254) of its first tile, so a
 *                        consumer's wait runs out, the kernel records a status code
 *                        (sm120_get_kernel_status) and returns; C is garbage
 *   TRACE                desc->workspace (>= SM120_TRACE_BYTES, 8-byte aligned)
 *                        receives a timeline of the launch, SM120_TRACE_WORDS_PER_CTA
 *                        64-bit words per CTA, CTA b at word b * WORDS_PER_CTA:
 *                          0 %globaltimer (ns) at kernel entry     1 %clock64 at entry
 *                          2 %globaltimer after set-up and the wait for the previous kernel    3 %clock64 then
 *                          4 %globaltimer at exit                  5 %clock64 at exit
 *                          6 tiles this CTA worked on              7 SM id
 *                          8 + 4 i + {0,1,2,3}, tile i < 8: %clock64 when the tile's first k-block had
 *                            landed / when its last MMA was issued (both: MMA warp, pair leader only) /
 *                            when its accumulator became readable / when its last store was committed
 *                            (both: first epilogue warp)
 *                        Not together with the FP32 tensor-core path, which needs the workspace itself.
 */
#define SM120_TUNE_CTA_GROUP_1     0x1
#define SM120_TUNE_CTA_GROUP_2     0x2
#define SM120_TUNE_EPI_WARPS_8     0x4
#define SM120_TUNE_EPI_WARPS_16    0x8
#define SM120_TUNE_NO_SPLIT_TAIL   0x10
#define SM120_TUNE_TRACE           0x20
#define SM120_TUNE_NO_SPLIT_K      0x40
#define SM120_TUNE_GROUP_M(g)      (((g) & 0xFF) << 8)
#define SM120_TUNE_STALL_KBLOCK(kb) ((((kb) + 1) & 0xFF) << 16)
#define SM120_TRACE_WORDS_PER_CTA  40
#define SM120_TRACE_MAX_CTAS       160
#define SM120_TRACE_BYTES          (SM120_TRACE_MAX_CTAS * SM120_TRACE_WORDS_PER_CTA * 8)

/* Fills *desc with defaults: struct_size, batch = 1, alpha = 1, beta = 0,
 * scales = 1, activation NONE, path AUTO, optimization_level = 1, all else 0. */
void sm120_gemm_desc_init(SM120GemmDesc* desc);

/* No counterpart in the reference: the launcher its OpKernels need
 * (see SM120GemmDesc above).  Same contract as sm120_launch_matmul. */
cudaError_t sm120_launch_matmul_ex(const SM120GemmDesc* desc);

/*
 * The product of sm120_launch_matmul_ex whose result block is ALSO written, by
 * the same kernel's epilogue, into up to 7 further buffers: peer_c[g] points
 * (in this process's address space) at the place of this [M, N] block inside
 * buffer g, which uses the same pitch (ldc), batch stride and dtype as desc->C.
 * With one process per GPU and the buffers living on the other GPUs of the box
 * (mapped through CUDA IPC, peer access enabled, see
 * sm120_enable_peer_access), this is the M-sharded product and its all-gather
 * in one launch: every rank's rows reach every rank's copy of C over NVLink
 * while the tiles are being computed, and no collective moves data afterwards.
 * The caller still has to order the ranks (any barrier) before reading rows
 * that other ranks wrote.  Requires the tensor-core path with beta == 0 and C,
 * ldc and every peer_c[g] 16-byte aligned; otherwise cudaErrorInvalidValue.
 * No counterpart in the reference, which has no multi-GPU code.
 */
cudaError_t sm120_launch_matmul_gather(const SM120GemmDesc* desc, void* const* peer_c, int num_peers);

/* Lets kernels launched on the current device write to memory of peer_device
 * (cudaDeviceEnablePeerAccess; already-enabled is not an error).
 * No counterpart in the reference. */
cudaError_t sm120_enable_peer_access(int peer_device);

/*
 * Sharing one rank's C buffer with the other processes of the box (CUDA IPC),
 * for sm120_launch_matmul_gather.  No counterpart in the reference.
 *   export: `ptr` is any device pointer of this process (e.g. inside a framework
 *     allocator's block); handle_out receives the 64-byte IPC handle of the
 *     allocation that contains it and *offset_out the byte offset of ptr in it.
 *   import: call with the device current whose kernels will write the memory;
 *     *base_out receives the address of the peer's allocation in this process
 *     (add the exporter's offset).  Peer access is set up by the import.
 *   close: unmaps an imported allocation.
 */
cudaError_t sm120_ipc_export(const void* ptr, void* handle_out, uint64_t* offset_out);
cudaError_t sm120_ipc_import(const void* handle, void** base_out);
cudaError_t sm120_ipc_close(void* base);

/*
 * Workspace for FP32 on the tensor cores (3xTF32: each operand is split into
 * two tf32 pieces by a pre-pass and three partial products are accumulated by
 * the tensor cores).  FLOAT32 inputs take this path when desc->workspace holds
 * at least the returned number of bytes (16-byte aligned) and either
 * desc->path == SM120_PATH_TENSOR_CORE (rejected without the workspace) or the
 * path is AUTO and the product has at least 2^24 multiply-adds; without
 * workspace AUTO runs the exact FFMA kernel.
 * Accuracy: the tensor cores truncate when they add into their fp32
 * accumulator, so a sum is carried there for 192 elements of K (3 x 192 tf32
 * products) only; the partial
 * sums are added in registers with round-to-nearest.  The relative Frobenius
 * error against float64 stays below 1e-5 (the op's fp32 gate) for K up to 8192,
 * same-sign data included; the FFMA kernel's stays below 1e-6.
 * FLOAT16 / BFLOAT16 / FP8 inputs: split-K.  A product whose output tiles would
 * occupy less than half of the GPU and whose K is long (at least 16 k-blocks of
 * 128 bytes) is cut into 2..8 consecutive K ranges that run as ONE tensor-core
 * launch into fp32 partial sums in the workspace; a second kernel adds the parts
 * in ascending order (reproducible, no atomics) and applies alpha, beta, bias,
 * activation and the output type.  The returned size is parts * M * N * 4 bytes
 * for such a product and 0 otherwise; a launch whose workspace is absent or
 * smaller runs unsplit.  Batched products, launches with peer destinations and
 * SM120_TUNE_NO_SPLIT_K are never split.
 * Returns 0 when the descriptor needs no workspace.  The workspace can
 * be reused by later calls on the same stream.  No counterpart in the reference.
 */
size_t sm120_matmul_workspace_bytes(const SM120GemmDesc* desc);

/*
 * Replaces LaunchSM120MatMulGradA / LaunchSM120MatMulGradB
 * (src/cuda_kernels/sm120_backward_kernels.cu:360-388; ops at
 * src/tensorflow_ops/sm120_gradients.cc:22-212), for an op
 * C = A[M,K] * B[K,N] without transposes:
 *   grad_a[M,K] = alpha * grad_c[M,N] * B[K,N]^T
 *   grad_b[K,N] = alpha * A[M,K]^T * grad_c[M,N]
 * All matrices row-major and dense, of type dtype.
 */
cudaError_t sm120_launch_matmul_grad_a(
    const void* grad_c, const void* B, void* grad_a,
    int M, int N, int K, float alpha,
    SM120DataType dtype, cudaStream_t stream);
cudaError_t sm120_launch_matmul_grad_b(
    const void* A, const void* grad_c, void* grad_b,
    int M, int N, int K, float alpha,
    SM120DataType dtype, cudaStream_t stream);

/*
 * Replaces sm120_launch_activation (src/cuda_kernels/sm120_c_interface.h:95-100,
 * body src/cuda_kernels/sm120_c_interface.cu:139-164, kernel
 * src/cuda_kernels/sm120_pure_kernels.cu:128-176) with the same signature:
 * output[i] = act(input[i]) for `size` elements of `dtype` (FLOAT32 or FLOAT16 as
 * in the reference, plus BFLOAT16), computed in fp32 and rounded to nearest.
 * Codes 0..8 are the reference's formulas, 9 is the erf GELU, and any other code
 * leaves the values unchanged, as the reference kernel's `default:` does.  A
 * dtype it does not know returns cudaErrorInvalidValue (:160-162).  In place
 * (output == input) is allowed.  This is the part of a Dense layer that remains
 * when its activation cannot be fused into the GEMM epilogue; it is bound by
 * HBM bandwidth (one read and one write of the tensor).
 */
cudaError_t sm120_launch_activation(
    const void* input, void* output,
    int size,
    SM120ActivationType activation_type,
    SM120DataType dtype,
    cudaStream_t stream);

/*
 * output[r, c] = act(input[r, c] + bias[c]) over a dense [rows, cols] matrix in one
 * pass: tf.nn.bias_add followed by the activation
 * (python/sm120_keras_layers.py:169-172) as ONE HBM-bound kernel, for outputs of
 * a matmul that was not launched with the fused epilogue.  bias has `cols`
 * entries of bias_dtype (FLOAT32 / FLOAT16 / BFLOAT16) or is null; sizes are 64-bit.
 * The reference has the activation launcher only (see above).
 */
cudaError_t sm120_launch_bias_activation(
    const void* input, const void* bias, SM120DataType bias_dtype, void* output,
    int64_t rows, int64_t cols,
    SM120ActivationType activation_type,
    SM120DataType dtype,
    cudaStream_t stream);

/*
 * Replaces sm120_launch_softmax (src/cuda_kernels/sm120_c_interface.h:189-195,
 * body src/cuda_kernels/sm120_c_interface.cu:374-400, kernel
 * src/cuda_kernels/sm120_pure_kernels.cu:471-550) with the same signature: softmax
 * over the middle extent of a dense [outer_size, axis_size, inner_size] tensor of
 * `dtype` (FLOAT32 / FLOAT16 as in the reference, plus BFLOAT16), fp32 math with
 * the maximum subtracted, in place allowed.  Rows of up to 8192 contiguous
 * elements (inner_size == 1) are read once and written once: the kernel is bound
 * by HBM bandwidth.
 */
cudaError_t sm120_launch_softmax(
    const void* logits, void* output,
    int outer_size, int axis_size, int inner_size,
    SM120DataType dtype,
    cudaStream_t stream);

/*
 * Row softmax with what the attention layer applies before it folded in
 * (python/sm120_ops.py:385-402, python/sm120_keras_layers.py:815-822):
 *   output[r, :] = softmax_c( scale * logits[r, c] + mask_factor * mask[r % mask_rows, c] )
 * over a dense [rows, cols] matrix of `dtype`, written as out_dtype (the same type,
 * or FLOAT16 / BFLOAT16 for FLOAT32 logits: fp32 scores in, 16-bit probabilities out
 * for the P.V product); `mask` (fp32, mask_rows x cols, device) may be
 * null; with causal != 0 column c of row r is excluded when
 * c > (r % seq_q) + cols - seq_q (rows are seq_q queries per batch entry, aligned
 * to the end of the cols keys).  A row with every column excluded comes out as
 * zeros.  No counterpart in the reference, which masks with separate TensorFlow ops.
 */
cudaError_t sm120_launch_softmax_ex(
    const void* logits, void* output,
    int64_t rows, int64_t cols,
    SM120DataType dtype, SM120DataType out_dtype, float scale,
    const float* mask, int64_t mask_rows, float mask_factor,
    int causal, int64_t seq_q,
    cudaStream_t stream);

/*
 * Replaces sm120_launch_attention (src/cuda_kernels/sm120_c_interface.h:138-144,
 * body src/cuda_kernels/sm120_c_interface.cu:232-268, kernel
 * src/cuda_kernels/sm120_pure_kernels.cu:352-430) with the same signature:
 *   output[b] = softmax(scale * Q[b] K[b]^T) V[b],   b < batch_size (batch x heads)
 * Q, K, V and output are dense [batch_size, seq_len, head_dim] tensors of `dtype`;
 * attention_weights is null or receives the fp32 [batch_size, seq_len, seq_len]
 * softmax.  FLOAT16 / BFLOAT16 with head_dim 64 or 128 run ONE fused tcgen05
 * kernel (scores and probabilities never reach HBM; when attention_weights is
 * requested it is produced beside it by a GEMM and a softmax pass).  FLOAT32
 * runs as GEMM + softmax + GEMM and uses attention_weights as its score matrix,
 * so it must be given; other combinations return cudaErrorInvalidValue.
 * The _ex form adds separate query and key lengths and the causal mask
 * (python/sm120_ops.py:388-398): key k of query q takes part when
 * k <= q + seq_k - seq_q.
 */
cudaError_t sm120_launch_attention(
    const void* queries, const void* keys, const void* values,
    void* output, float* attention_weights,
    int batch_size, int seq_len, int head_dim,
    float scale,
    SM120DataType dtype,
    cudaStream_t stream);
cudaError_t sm120_launch_attention_ex(
    const void* queries, const void* keys, const void* values,
    void* output, float* attention_weights,
    int64_t batch_size, int64_t seq_q, int64_t seq_k, int64_t head_dim,
    float scale, int causal,
    SM120DataType dtype,
    cudaStream_t stream);

/*
 * Bias gradient of the Dense layer: grad_bias[n] = sum over m of grad_c[m, n] for a
 * row-major [M, N] matrix with row pitch ld (elements; 0 = N), accumulated in fp32
 * in a fixed order (bitwise reproducible; no atomics, no scratch) and written as
 * out_dtype (FLOAT32, or the same type as grad_c).  It completes the backward
 * pass next to sm120_launch_matmul_grad_a / _b: the reference's layer adds its
 * bias with tf.nn.bias_add (python/sm120_keras_layers.py:169), whose gradient is
 * this column sum; the reference's own gradient ops
 * (src/tensorflow_ops/sm120_gradients.cc:22-212) cover the two matmuls only.
 */
cudaError_t sm120_launch_bias_grad(
    const void* grad_c, void* grad_bias,
    int64_t M, int64_t N, int64_t ld,
    SM120DataType dtype, SM120DataType out_dtype,
    cudaStream_t stream);

/*
 * Per-tensor FP8 quantisation, the producer of FP8 matmul operands:
 *   *scale_out = 448 / max|x|   (1 for an all-zero tensor)
 *   q[i] = saturate_e4m3(x[i] * *scale_out)      (round-to-nearest-even, finite)
 * Non-finite input: an infinity enters the maximum as the largest finite float, so
 * the scale stays positive and finite (the infinity saturates to +-448, finite
 * values become 0); a NaN is ignored by the maximum and comes out as the e4m3 NaN.
 * x has n elements of x_dtype (FLOAT32, FLOAT16 or BFLOAT16); q receives n bytes;
 * scale_out is one float in device memory and can be passed straight to
 * SM120GemmDesc::scale_a_dev / scale_b_dev.  `scratch` is device memory of at
 * least sm120_quantize_fp8_scratch_bytes(n) bytes (4 bytes per 65536 elements),
 * 4-byte aligned, owned by the caller; its contents before the call do not
 * matter and it may be reused by the next call on the same stream.
 * The reference declares the FP8 type and its saturating conversion
 * (src/cuda_kernels/sm120_datatype_support.h:71-82,168-171;
 * python/sm120_datatype_manager.py:88-98) but has no launcher that produces
 * FP8 tensors; this is that launcher.
 */
size_t sm120_quantize_fp8_scratch_bytes(int64_t n);
cudaError_t sm120_launch_quantize_fp8(
    const void* x, SM120DataType x_dtype, int64_t n,
    void* q, float* scale_out,
    void* scratch, size_t scratch_bytes,
    cudaStream_t stream);

/*
 * Only the cast of the quantisation above, with a scale the caller already has:
 * q[i] = saturate_e4m3(x[i] * *scale), `scale` one float in device memory.  For a
 * tensor that is sharded over several GPUs, whose scale comes from the maximum
 * over all shards, so that every rank quantises with the same number.  Needs no
 * scratch.  No counterpart in the reference (see sm120_launch_quantize_fp8).
 */
cudaError_t sm120_launch_cast_fp8(
    const void* x, SM120DataType x_dtype, int64_t n,
    const float* scale, void* q,
    cudaStream_t stream);

/*
 * The same quantisation for callers that cannot hand over scratch memory.
 * It has no counterpart in the reference.
 *
 * Who needs it: code that runs where asking the device for memory is off the
 * table -- a framework callback that may touch only the tensors the framework
 * passed in, a serving loop that fixed its memory pool at start-up, a
 * foreign-language binding that owns no device buffers.  Such a caller still
 * passes its input, its output and the float that receives the scale; the
 * partial maxima that sm120_launch_quantize_fp8 keeps in `scratch` go into a
 * 16 KB array that is part of this library's device image instead (every GPU
 * that loads the library carries it until the process ends).  The call itself
 * performs no cudaMalloc / cudaFree and uses no allocating library routine.
 *
 * Limit: n <= SM120_QUANTIZE_FP8_STATIC_MAX_ELEMENTS (268 435 456); a larger n
 * is rejected with cudaErrorInvalidValue before anything is launched -- use
 * sm120_launch_quantize_fp8 with your own scratch for bigger tensors.
 *
 * First call on a device: the library looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and remembers it.  Make that
 * first call ahead of any stream capture.
 *
 * Sharing: every call on a device uses the same array, which keeps whatever the
 * previous call left in it.  That is harmless -- each slot a call reads is
 * written by that call first, nothing has to start at zero -- but two calls
 * that overlap on the GPU (different streams, no ordering between them) would
 * overwrite each other's partial maxima: order them, or use the scratch-taking
 * entry point for concurrent work.
 */
#define SM120_QUANTIZE_FP8_STATIC_MAX_ELEMENTS 268435456ll
cudaError_t sm120_launch_quantize_fp8_static(
    const void* x, SM120DataType x_dtype, int64_t n,
    void* q, float* scale_out,
    cudaStream_t stream);

/*
 * Replaces sm120_is_supported (src/cuda_kernels/sm120_c_interface.h:153, body
 * src/cuda_kernels/sm120_c_interface.cu:285-293, which accepts only compute
 * capability 12.0).  This build accepts compute capability 10.x (B200).
 */
bool sm120_is_supported(int device_id);

/* Replaces sm120_get_error_string (src/cuda_kernels/sm120_c_interface.h:209). */
const char* sm120_get_error_string(cudaError_t error);

/*
 * Device-side wait status.  Every wait inside the tcgen05 kernel (on a TMA
 * arrival, a free shared-memory stage or a TMEM accumulator) is bounded by a
 * wall-clock limit; a kernel that gives up records a non-zero code in a
 * per-device status word, drains and returns normally.  This call copies the
 * word for `device_id` to *status (0 = no timeout seen) and, when `clear` is
 * non-zero, resets it.  It synchronises the device.  The reference has no
 * counterpart; its closest relative is SM120ErrorHandler
 * (src/cuda_kernels/sm120_error_handling.cu:48-94), which only logs.
 */
cudaError_t sm120_get_kernel_status(int device_id, unsigned int* status, int clear);

/*
 * Clock seen from inside the most recent tensor-core launch on `device_id`:
 * *cycles = SM cycles (%clock64) and *ns = nanoseconds (%globaltimer) that CTA 0
 * of that launch was alive; cycles / ns is the SM clock in GHz under the load the
 * kernel itself produced (a power-capped part runs well below its maximum).  It
 * synchronises the device.  Two launches in flight at once overwrite each
 * other's two words; nothing else depends on them.  No counterpart in the reference.
 */
cudaError_t sm120_get_kernel_clock(int device_id, unsigned long long* cycles, unsigned long long* ns);

/*
 * TMA tensor maps (three per tensor-core launch) are cached per host thread,
 * keyed by address, type, extents, pitches and box; this reports how many the
 * process has encoded through the driver and how many launches reused a cached
 * one.  Either pointer may be null.  No counterpart in the reference.
 */
void sm120_get_tensor_map_stats(uint64_t* encoded, uint64_t* reused);

/* Wait limit, in milliseconds, used by launches made after the call
 * (default 2000; also read once from the environment variable
 * SM120_WAIT_LIMIT_MS).  No counterpart in the reference. */
void sm120_set_wait_limit_ms(unsigned int ms);

/* Number of kernels this library has enqueued since it was loaded
 * (both families).  No counterpart in the reference; used to count launches
 * inside a timed region. */
uint64_t sm120_get_launch_count(void);

/* Name of the kernel variant the last launch on this host thread used, e.g.
 * "tc_bf16_128x256x64_s4" or "simt_f32_64x64"; "" before any launch.
 * No counterpart in the reference. */
const char* sm120_get_last_kernel_name(void);

/* Number of K ranges (1 = not split) of the last matmul launch on this host
 * thread.  No counterpart in the reference. */
int sm120_get_last_split_k(void);

#ifdef __cplusplus
}
#endif

#endif /* SM120_C_INTERFACE_H */
