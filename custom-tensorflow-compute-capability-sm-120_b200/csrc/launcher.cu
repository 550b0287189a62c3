// C ABI of the SM120 matmul op for B200: argument validation, defaults, choice
// of kernel family, and the entry points declared in include/sm120_c_interface.h.
// Mirrors the role of src/cuda_kernels/sm120_c_interface.cu:32-60 in the
// reference (grid choice + dtype dispatch + cudaGetLastError()).
//
// The launchers hold no mutable global state except monotonic counters,
// per-device caches of immutable device attributes and each thread's own cache
// of tensor maps, so they may be called concurrently from any number of host
// threads; everything that varies per call travels in the descriptor.

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <atomic>

#include "gemm_common.h"

namespace sm120 {

long long quant_spans(long long n);
cudaError_t quant_launch(const void* x, int x_dtype, void* q, float* scale_out, long long n, float* partial, cudaStream_t stream);
cudaError_t quant_launch_static(const void* x, int x_dtype, void* q, float* scale_out, long long n, int device, cudaStream_t stream);
cudaError_t quant_cast_launch(const void* x, int x_dtype, void* q, const float* scale, long long n, cudaStream_t stream);
cudaError_t activation_launch(const void* in, void* out, long long n, const void* bias, int bias_dtype, long long cols,
                              int act, int dtype, int sm_count, cudaStream_t stream);
cudaError_t softmax_launch(const void* in, void* out, long long outer, long long axis, long long inner, int dtype, int out_dtype,
                           float scale, const float* mask, long long mask_rows, float mask_factor, int causal, long long seq_q,
                           int sm_count, cudaStream_t stream);
bool attention_fused_supported(int dtype, long long batch, long long seq_q, long long seq_k, long long head_dim, const void* q,
                               const void* k, const void* v, const void* out);
cudaError_t attention_fused_launch(const void* q, const void* k, const void* v, void* out, long long batch, long long seq_q,
                                   long long seq_k, long long head_dim, float scale, int causal, int dtype, int device,
                                   uint64_t wait_limit_ns, cudaStream_t stream);
cudaError_t bias_grad_launch(const void* g, int dtype, long long M, long long N, long long ld, void* out, int out_dtype,
                             cudaStream_t stream);

namespace {

constexpr int MAX_DEVICES = 64;

struct DeviceInfo {
    std::atomic<int> state{0};   // 0 unknown, 1 supported, 2 unsupported
    std::atomic<int> sm_count{0};
};
DeviceInfo g_devices[MAX_DEVICES];

std::atomic<uint64_t> g_launch_count{0};
std::atomic<uint64_t> g_wait_limit_ns{0};   // 0 = not initialised yet
thread_local const char* t_last_kernel = "";
thread_local int t_last_split_k = 1;        // K parts of this thread's last matmul launch

uint64_t wait_limit_ns() {
    uint64_t v = g_wait_limit_ns.load(std::memory_order_relaxed);
    if (v != 0) return v;
    uint64_t ms = 2000;
    const char* env = getenv("SM120_WAIT_LIMIT_MS");
    if (env != nullptr && env[0] != '\0') {
        const long parsed = strtol(env, nullptr, 10);
        if (parsed > 0) ms = static_cast<uint64_t>(parsed);
    }
    v = ms * 1000000ull;
    g_wait_limit_ns.store(v, std::memory_order_relaxed);
    return v;
}

// Returns cudaSuccess and fills sm_count when `device` is a compute-capability 10.x part.
cudaError_t query_device(int device, int* sm_count) {
    if (device < 0 || device >= MAX_DEVICES) return cudaErrorInvalidDevice;
    DeviceInfo& d = g_devices[device];
    int st = d.state.load(std::memory_order_acquire);
    if (st == 0) {
        int major = 0, sms = 0;
        cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return e;
        d.sm_count.store(sms, std::memory_order_relaxed);
        st = (major == 10) ? 1 : 2;
        d.state.store(st, std::memory_order_release);
    }
    if (st != 1) return cudaErrorInvalidDevice;
    *sm_count = d.sm_count.load(std::memory_order_relaxed);
    return cudaSuccess;
}

bool valid_dtype(int d) { return d >= SM120_DTYPE_FLOAT32 && d <= SM120_DTYPE_FP8_E4M3; }

// Checks every field that can be checked without touching the device and
// resolves defaults.  Returns cudaErrorInvalidValue for a rejected descriptor.
cudaError_t resolve(const SM120GemmDesc* d, GemmProblem* out) {
    if (d == nullptr) return cudaErrorInvalidValue;
    if (d->struct_size != sizeof(SM120GemmDesc)) return cudaErrorInvalidValue;
    if (!valid_dtype(d->in_dtype) || !valid_dtype(d->out_dtype)) return cudaErrorInvalidValue;
    if (d->out_dtype == SM120_DTYPE_FP8_E4M3) return cudaErrorInvalidValue;
    if (d->M < 0 || d->N < 0 || d->K < 0 || d->batch < 1) return cudaErrorInvalidValue;
    if (d->activation < SM120_ACTIVATION_NONE || d->activation > SM120_ACTIVATION_GELU_ERF) return cudaErrorInvalidValue;
    if (d->path < SM120_PATH_AUTO || d->path > SM120_PATH_SIMT) return cudaErrorInvalidValue;
    if (d->optimization_level < 0 || d->optimization_level > 2) return cudaErrorInvalidValue;
    if (d->bias != nullptr) {
        if (d->bias_dtype != SM120_DTYPE_FLOAT32 && d->bias_dtype != SM120_DTYPE_FLOAT16 && d->bias_dtype != SM120_DTYPE_BFLOAT16)
            return cudaErrorInvalidValue;
    }
    if (d->scale_a < 0.0f || d->scale_b < 0.0f) return cudaErrorInvalidValue;
    if ((d->tuning & ~0x00FFFF7F) != 0) return cudaErrorInvalidValue;
    if ((d->tuning & SM120_TUNE_CTA_GROUP_1) && (d->tuning & SM120_TUNE_CTA_GROUP_2)) return cudaErrorInvalidValue;
    if ((d->tuning & SM120_TUNE_EPI_WARPS_8) && (d->tuning & SM120_TUNE_EPI_WARPS_16)) return cudaErrorInvalidValue;
    if (d->tuning & SM120_TUNE_TRACE) {
        if (d->workspace == nullptr || (reinterpret_cast<uintptr_t>(d->workspace) & 7u) != 0 || d->workspace_bytes < SM120_TRACE_BYTES)
            return cudaErrorInvalidValue;
        if (d->in_dtype == SM120_DTYPE_FLOAT32 && d->path == SM120_PATH_TENSOR_CORE) return cudaErrorInvalidValue;
    }

    GemmProblem p{};
    p.M = d->M; p.N = d->N; p.K = d->K; p.batch = d->batch;
    p.transpose_a = d->transpose_a != 0; p.transpose_b = d->transpose_b != 0;
    const int64_t a_row = p.transpose_a ? p.M : p.K;     // stored row length of A
    const int64_t a_rows = p.transpose_a ? p.K : p.M;
    const int64_t b_row = p.transpose_b ? p.K : p.N;
    const int64_t b_rows = p.transpose_b ? p.N : p.K;
    p.lda = d->lda != 0 ? d->lda : a_row;
    p.ldb = d->ldb != 0 ? d->ldb : b_row;
    p.ldc = d->ldc != 0 ? d->ldc : p.N;
    if (p.lda < a_row || p.ldb < b_row || p.ldc < p.N) return cudaErrorInvalidValue;
    if (d->stride_a < 0 || d->stride_b < 0 || d->stride_c < 0) return cudaErrorInvalidValue;
    p.stride_a = d->stride_a; p.stride_b = d->stride_b; p.stride_c = d->stride_c;
    if (p.batch > 1) {
        // C entries must not overlap; A and B may broadcast with stride 0
        if (p.stride_c < (p.M > 0 ? (p.M - 1) * p.ldc + p.N : 0)) return cudaErrorInvalidValue;
        if (p.stride_a != 0 && p.stride_a < (a_rows > 0 ? (a_rows - 1) * p.lda + a_row : 0)) return cudaErrorInvalidValue;
        if (p.stride_b != 0 && p.stride_b < (b_rows > 0 ? (b_rows - 1) * p.ldb + b_row : 0)) return cudaErrorInvalidValue;
    }
    const bool empty_out = (p.M == 0 || p.N == 0);
    if (!empty_out) {
        if (d->C == nullptr) return cudaErrorInvalidValue;
        if (p.K > 0 && (d->A == nullptr || d->B == nullptr)) return cudaErrorInvalidValue;
    }
    p.A = d->A; p.B = d->B; p.C = d->C; p.bias = d->bias;
    p.in_dtype = d->in_dtype; p.out_dtype = d->out_dtype; p.bias_dtype = d->bias_dtype;
    p.alpha = d->alpha; p.beta = d->beta;
    const float sa = d->scale_a == 0.0f ? 1.0f : d->scale_a;
    const float sb = d->scale_b == 0.0f ? 1.0f : d->scale_b;
    p.inv_scale = 1.0f / (sa * sb);
    p.scale_a_dev = d->scale_a_dev; p.scale_b_dev = d->scale_b_dev;
    p.activation = d->activation;
    p.optimization_level = d->optimization_level;
    p.tuning = d->tuning;
    p.trace = (d->tuning & SM120_TUNE_TRACE) ? d->workspace : nullptr;
    p.stream = d->stream;
    *out = p;
    return cudaSuccess;
}

cudaError_t launch_resolved(GemmProblem& p, int path, void* workspace = nullptr, uint64_t workspace_bytes = 0) {
    if (p.M == 0 || p.N == 0) return cudaSuccess;    // nothing to write
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    int sms = 0;
    e = query_device(device, &sms);
    if (e != cudaSuccess) return e;
    p.device = device;
    p.sm_count = sms;

    const char* why = nullptr;
    const char* name = "";
    // FP32 on the tensor cores (3xTF32) needs workspace for the split operands.  A forced tensor-core launch
    // without it is rejected; AUTO takes the tensor cores when the caller supplied enough workspace and the
    // product is large enough to repay the two split passes, and the exact FFMA kernel otherwise.
    const bool fp32_ws = p.in_dtype == SM120_DTYPE_FLOAT32 && p.trace == nullptr && p.K >= 1 && workspace != nullptr &&
                         (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0 && workspace_bytes >= tf32x3_workspace_bytes(p);
    const bool fp32_big = static_cast<double>(p.M) * static_cast<double>(p.N) * static_cast<double>(p.K) * static_cast<double>(p.batch) >= 16777216.0;
    if (p.in_dtype == SM120_DTYPE_FLOAT32 && (path == SM120_PATH_TENSOR_CORE || (path == SM120_PATH_AUTO && fp32_ws && fp32_big))) {
        if (!fp32_ws) return cudaErrorInvalidValue;
        e = tf32x3_launch(p, workspace, wait_limit_ns(), &name);
        if (e == cudaErrorInvalidValue && path == SM120_PATH_AUTO) {
            // the split operands cannot be described to TMA (extents beyond its limits): nothing was enqueued
            e = simt_launch(p, &name);
            if (e == cudaSuccess) {
                g_launch_count.fetch_add(1, std::memory_order_relaxed);
                t_last_kernel = name;
            }
            return e;
        }
        if (e == cudaSuccess) {
            g_launch_count.fetch_add(2, std::memory_order_relaxed);
            t_last_kernel = name;
        }
        return e;
    }
    const bool tc_ok = tc_supported(p, &why);
    if (path == SM120_PATH_TENSOR_CORE && !tc_ok) return cudaErrorInvalidValue;
    // few output tiles and a long K: split K over the idle SMs when the caller gave workspace for the partial sums
    if (path != SM120_PATH_SIMT && tc_ok && workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0) {
        const size_t need = splitk_workspace_bytes(p);
        if (need != 0 && workspace_bytes >= need) {
            e = splitk_launch(p, workspace, wait_limit_ns(), &name);
            if (e == cudaSuccess) {
                g_launch_count.fetch_add(2, std::memory_order_relaxed);
                t_last_kernel = name;
                t_last_split_k = splitk_factor(p);
                return e;
            }
            if (e != cudaErrorInvalidValue) return e;          // InvalidValue: nothing was enqueued; run unsplit
        }
    }
    t_last_split_k = 1;
    if (path != SM120_PATH_SIMT && tc_ok) {
        e = tc_launch(p, wait_limit_ns(), &name);
    } else {
        e = simt_launch(p, &name);
    }
    if (e == cudaSuccess) {
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
        t_last_kernel = name;
    }
    return e;
}

}  // namespace
}  // namespace sm120

using namespace sm120;

extern "C" {

void sm120_gemm_desc_init(SM120GemmDesc* desc) {
    if (desc == nullptr) return;
    memset(desc, 0, sizeof(*desc));
    desc->struct_size = sizeof(SM120GemmDesc);
    desc->batch = 1;
    desc->alpha = 1.0f;
    desc->beta = 0.0f;
    desc->scale_a = 1.0f;
    desc->scale_b = 1.0f;
    desc->activation = SM120_ACTIVATION_NONE;
    desc->path = SM120_PATH_AUTO;
    desc->optimization_level = 1;
}

cudaError_t sm120_launch_matmul_ex(const SM120GemmDesc* desc) {
    GemmProblem p;
    cudaError_t e = resolve(desc, &p);
    if (e != cudaSuccess) return e;
    return launch_resolved(p, desc->path, desc->workspace, desc->workspace_bytes);
}

cudaError_t sm120_launch_matmul_gather(const SM120GemmDesc* desc, void* const* peer_c, int num_peers) {
    GemmProblem p;
    cudaError_t e = resolve(desc, &p);
    if (e != cudaSuccess) return e;
    if (num_peers < 0 || num_peers > 7 || (num_peers > 0 && peer_c == nullptr)) return cudaErrorInvalidValue;
    if (p.beta != 0.0f || p.in_dtype == SM120_DTYPE_FLOAT32) return cudaErrorInvalidValue;
    for (int g = 0; g < num_peers; ++g) {
        if (peer_c[g] == nullptr) return cudaErrorInvalidValue;
        p.extra_dests[g] = peer_c[g];
    }
    p.num_extra_dests = num_peers;
    return launch_resolved(p, SM120_PATH_TENSOR_CORE);
}

cudaError_t sm120_enable_peer_access(int peer_device) {
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();       // clear the sticky-less error state
        return cudaSuccess;
    }
    return e;
}

cudaError_t sm120_ipc_export(const void* ptr, void* handle_out, uint64_t* offset_out) {
    if (ptr == nullptr || handle_out == nullptr || offset_out == nullptr) return cudaErrorInvalidValue;
    // base of the allocation that holds ptr (driver call, resolved at run time: no link-time dependency on libcuda)
    typedef int (*GetRangeFn)(unsigned long long*, size_t*, unsigned long long);
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q);
    if (e != cudaSuccess) return e;
    if (q != cudaDriverEntryPointSuccess || sym == nullptr) return cudaErrorNotSupported;
    unsigned long long base = 0;
    size_t size = 0;
    if (reinterpret_cast<GetRangeFn>(sym)(&base, &size, reinterpret_cast<unsigned long long>(ptr)) != 0) return cudaErrorInvalidValue;
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
    if (e != cudaSuccess) return e;
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle_out, &h, sizeof(h));
    *offset_out = reinterpret_cast<unsigned long long>(ptr) - base;
    return cudaSuccess;
}

cudaError_t sm120_ipc_import(const void* handle, void** base_out) {
    if (handle == nullptr || base_out == nullptr) return cudaErrorInvalidValue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* base = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return e;
    cudaPointerAttributes attr;
    e = cudaPointerGetAttributes(&attr, base);
    if (e != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
        cudaIpcCloseMemHandle(base);
        return e != cudaSuccess ? e : cudaErrorInvalidValue;
    }
    *base_out = base;
    return cudaSuccess;
}

cudaError_t sm120_ipc_close(void* base) {
    if (base == nullptr) return cudaErrorInvalidValue;
    return cudaIpcCloseMemHandle(base);
}

size_t sm120_matmul_workspace_bytes(const SM120GemmDesc* desc) {
    GemmProblem p;
    if (resolve(desc, &p) != cudaSuccess) return 0;
    if (p.M == 0 || p.N == 0 || p.K == 0) return 0;
    if (p.in_dtype == SM120_DTYPE_FLOAT32) return tf32x3_workspace_bytes(p);
    // 16-bit and FP8 products take workspace only when they would be split along K
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || query_device(device, &sms) != cudaSuccess) return 0;
    p.device = device;
    p.sm_count = sms;
    const char* why = nullptr;
    if (desc->path == SM120_PATH_SIMT || !tc_supported(p, &why)) return 0;
    return splitk_workspace_bytes(p);
}

cudaError_t sm120_launch_matmul(const void* A, const void* B, void* C, int M, int N, int K, float alpha, float beta,
                                SM120DataType dtype, cudaStream_t stream) {
    // the reference launcher knows FLOAT32 and FLOAT16 and rejects the rest; BFLOAT16 is added, FP8 has no
    // same-type output and is rejected here
    if (dtype != SM120_DTYPE_FLOAT32 && dtype != SM120_DTYPE_FLOAT16 && dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    SM120GemmDesc d;
    sm120_gemm_desc_init(&d);
    d.A = A; d.B = B; d.C = C;
    d.M = M; d.N = N; d.K = K;
    d.alpha = alpha; d.beta = beta;
    d.in_dtype = dtype; d.out_dtype = dtype;
    d.stream = stream;
    return sm120_launch_matmul_ex(&d);
}

void launch_sm120_matmul(const float* A, const float* B, float* C, int M, int N, int K, cudaStream_t stream) {
    (void)sm120_launch_matmul(A, B, C, M, N, K, 1.0f, 0.0f, SM120_DTYPE_FLOAT32, stream);
}

cudaError_t sm120_launch_matmul_grad_a(const void* grad_c, const void* B, void* grad_a, int M, int N, int K, float alpha,
                                       SM120DataType dtype, cudaStream_t stream) {
    if (dtype != SM120_DTYPE_FLOAT32 && dtype != SM120_DTYPE_FLOAT16 && dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    // grad_a[M,K] = grad_c[M,N] * B[K,N]^T : a GEMM with inner dimension N and B read transposed
    SM120GemmDesc d;
    sm120_gemm_desc_init(&d);
    d.A = grad_c; d.B = B; d.C = grad_a;
    d.M = M; d.N = K; d.K = N;
    d.transpose_b = 1;
    d.alpha = alpha;
    d.in_dtype = dtype; d.out_dtype = dtype;
    d.stream = stream;
    return sm120_launch_matmul_ex(&d);
}

cudaError_t sm120_launch_matmul_grad_b(const void* A, const void* grad_c, void* grad_b, int M, int N, int K, float alpha,
                                       SM120DataType dtype, cudaStream_t stream) {
    if (dtype != SM120_DTYPE_FLOAT32 && dtype != SM120_DTYPE_FLOAT16 && dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    // grad_b[K,N] = A[M,K]^T * grad_c[M,N] : a GEMM with inner dimension M and A read transposed
    SM120GemmDesc d;
    sm120_gemm_desc_init(&d);
    d.A = A; d.B = grad_c; d.C = grad_b;
    d.M = K; d.N = N; d.K = M;
    d.transpose_a = 1;
    d.alpha = alpha;
    d.in_dtype = dtype; d.out_dtype = dtype;
    d.stream = stream;
    return sm120_launch_matmul_ex(&d);
}

size_t sm120_quantize_fp8_scratch_bytes(int64_t n) {
    return n > 0 ? static_cast<size_t>(quant_spans(n)) * sizeof(float) : 0;
}

cudaError_t sm120_launch_quantize_fp8(const void* x, SM120DataType x_dtype, int64_t n, void* q, float* scale_out,
                                      void* scratch, size_t scratch_bytes, cudaStream_t stream) {
    if (n < 0 || scale_out == nullptr) return cudaErrorInvalidValue;
    if (x_dtype != SM120_DTYPE_FLOAT32 && x_dtype != SM120_DTYPE_FLOAT16 && x_dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    if (n > 0 && (x == nullptr || q == nullptr || scratch == nullptr)) return cudaErrorInvalidValue;
    if (scratch_bytes < sm120_quantize_fp8_scratch_bytes(n)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(scratch) & 3u) != 0 || (reinterpret_cast<uintptr_t>(scale_out) & 3u) != 0)
        return cudaErrorInvalidValue;
    if (n == 0) return cudaSuccess;
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    e = query_device(device, &sms);
    if (e != cudaSuccess) return e;
    e = quant_launch(x, x_dtype, q, scale_out, n, static_cast<float*>(scratch), stream);
    if (e == cudaSuccess) {
        g_launch_count.fetch_add(2, std::memory_order_relaxed);
        t_last_kernel = "quant_e4m3_amax_scale_cast";
    }
    return e;
}

// Quantisation without caller scratch and without any allocation: the partial
// maxima go to a fixed array inside the library (see the header for who needs
// this, the size limit, the first-call set-up and the sharing rule).
cudaError_t sm120_launch_quantize_fp8_static(const void* x, SM120DataType x_dtype, int64_t n, void* q, float* scale_out,
                                             cudaStream_t stream) {
    if (n < 0 || scale_out == nullptr) return cudaErrorInvalidValue;
    if (n > SM120_QUANTIZE_FP8_STATIC_MAX_ELEMENTS) return cudaErrorInvalidValue;     // beyond the built-in scratch
    if (x_dtype != SM120_DTYPE_FLOAT32 && x_dtype != SM120_DTYPE_FLOAT16 && x_dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    if (n > 0 && (x == nullptr || q == nullptr)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(scale_out) & 3u) != 0) return cudaErrorInvalidValue;
    if (n == 0) return cudaSuccess;
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    e = query_device(device, &sms);
    if (e != cudaSuccess) return e;
    e = quant_launch_static(x, x_dtype, q, scale_out, n, device, stream);
    if (e == cudaSuccess) {
        g_launch_count.fetch_add(2, std::memory_order_relaxed);
        t_last_kernel = "quant_e4m3_amax_scale_cast_static";
    }
    return e;
}

cudaError_t sm120_launch_cast_fp8(const void* x, SM120DataType x_dtype, int64_t n, const float* scale, void* q,
                                  cudaStream_t stream) {
    if (n < 0 || scale == nullptr) return cudaErrorInvalidValue;
    if (x_dtype != SM120_DTYPE_FLOAT32 && x_dtype != SM120_DTYPE_FLOAT16 && x_dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    if (n > 0 && (x == nullptr || q == nullptr)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(scale) & 3u) != 0) return cudaErrorInvalidValue;
    if (n == 0) return cudaSuccess;
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    e = query_device(device, &sms);
    if (e != cudaSuccess) return e;
    e = quant_cast_launch(x, x_dtype, q, scale, n, stream);
    if (e == cudaSuccess) {
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
        t_last_kernel = "quant_e4m3_scale_cast";
    }
    return e;
}

namespace {
cudaError_t activation_common(const void* input, const void* bias, int bias_dtype, void* output, int64_t rows, int64_t cols,
                              int activation_type, int dtype, cudaStream_t stream, const char* name) {
    if (rows < 0 || cols < 0) return cudaErrorInvalidValue;
    if (dtype != SM120_DTYPE_FLOAT32 && dtype != SM120_DTYPE_FLOAT16 && dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    if (bias != nullptr && bias_dtype != SM120_DTYPE_FLOAT32 && bias_dtype != SM120_DTYPE_FLOAT16 && bias_dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    if (cols != 0 && rows > INT64_MAX / cols) return cudaErrorInvalidValue;
    const int64_t n = rows * cols;
    if (n > 0 && (input == nullptr || output == nullptr)) return cudaErrorInvalidValue;
    if (n == 0) return cudaSuccess;
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    e = query_device(device, &sms);
    if (e != cudaSuccess) return e;
    e = activation_launch(input, output, n, bias, bias_dtype, cols, activation_type, dtype, sms, stream);
    if (e == cudaSuccess) {
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
        t_last_kernel = name;
    }
    return e;
}
}  // namespace

cudaError_t sm120_launch_activation(const void* input, void* output, int size, SM120ActivationType activation_type,
                                    SM120DataType dtype, cudaStream_t stream) {
    return activation_common(input, nullptr, 0, output, 1, size, static_cast<int>(activation_type), static_cast<int>(dtype),
                             stream, "activation_vec16");
}

cudaError_t sm120_launch_bias_activation(const void* input, const void* bias, SM120DataType bias_dtype, void* output,
                                         int64_t rows, int64_t cols, SM120ActivationType activation_type, SM120DataType dtype,
                                         cudaStream_t stream) {
    return activation_common(input, bias, static_cast<int>(bias_dtype), output, rows, cols, static_cast<int>(activation_type),
                             static_cast<int>(dtype), stream, bias != nullptr ? "bias_activation_vec16" : "activation_vec16");
}

cudaError_t sm120_launch_bias_grad(const void* grad_c, void* grad_bias, int64_t M, int64_t N, int64_t ld, SM120DataType dtype,
                                   SM120DataType out_dtype, cudaStream_t stream) {
    if (M < 0 || N < 0) return cudaErrorInvalidValue;
    if (dtype != SM120_DTYPE_FLOAT32 && dtype != SM120_DTYPE_FLOAT16 && dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    if (out_dtype != SM120_DTYPE_FLOAT32 && out_dtype != dtype) return cudaErrorInvalidValue;
    if (ld == 0) ld = N;
    if (ld < N) return cudaErrorInvalidValue;
    if (N > 0 && grad_bias == nullptr) return cudaErrorInvalidValue;
    if (N > 0 && M > 0 && grad_c == nullptr) return cudaErrorInvalidValue;
    if (N == 0) return cudaSuccess;
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    e = query_device(device, &sms);
    if (e != cudaSuccess) return e;
    e = bias_grad_launch(grad_c, dtype, M, N, ld, grad_bias, out_dtype, stream);     // M == 0 writes zeros
    if (e == cudaSuccess) {
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
        t_last_kernel = "bias_grad_colsum";
    }
    return e;
}

namespace {
cudaError_t softmax_common(const void* logits, void* output, int64_t outer, int64_t axis, int64_t inner, int dtype, int out_dtype, float scale,
                           const float* mask, int64_t mask_rows, float mask_factor, int causal, int64_t seq_q, cudaStream_t stream) {
    if (outer < 0 || axis < 0 || inner < 0) return cudaErrorInvalidValue;
    if (dtype != SM120_DTYPE_FLOAT32 && dtype != SM120_DTYPE_FLOAT16 && dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    if (out_dtype != dtype && !(dtype == SM120_DTYPE_FLOAT32 && (out_dtype == SM120_DTYPE_FLOAT16 || out_dtype == SM120_DTYPE_BFLOAT16)))
        return cudaErrorInvalidValue;
    if ((mask != nullptr || causal) && inner != 1) return cudaErrorInvalidValue;
    if (mask != nullptr && (mask_rows < 1 || (reinterpret_cast<uintptr_t>(mask) & 3u) != 0)) return cudaErrorInvalidValue;
    if (causal && (seq_q < 1 || seq_q > axis || (outer % seq_q) != 0)) return cudaErrorInvalidValue;
    if (outer == 0 || axis == 0 || inner == 0) return cudaSuccess;
    if (logits == nullptr || output == nullptr) return cudaErrorInvalidValue;
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    e = query_device(device, &sms);
    if (e != cudaSuccess) return e;
    e = softmax_launch(logits, output, outer, axis, inner, dtype, out_dtype, scale, mask, mask_rows, mask_factor, causal, seq_q, sms, stream);
    if (e == cudaSuccess) {
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
        t_last_kernel = "softmax_rows";
    }
    return e;
}
}  // namespace

cudaError_t sm120_launch_softmax(const void* logits, void* output, int outer_size, int axis_size, int inner_size,
                                 SM120DataType dtype, cudaStream_t stream) {
    return softmax_common(logits, output, outer_size, axis_size, inner_size, static_cast<int>(dtype), static_cast<int>(dtype), 1.0f, nullptr, 0, 0.0f, 0, 0, stream);
}

cudaError_t sm120_launch_softmax_ex(const void* logits, void* output, int64_t rows, int64_t cols, SM120DataType dtype,
                                    SM120DataType out_dtype, float scale, const float* mask, int64_t mask_rows, float mask_factor,
                                    int causal, int64_t seq_q, cudaStream_t stream) {
    return softmax_common(logits, output, rows, cols, 1, static_cast<int>(dtype), static_cast<int>(out_dtype), scale, mask, mask_rows, mask_factor, causal, seq_q, stream);
}

cudaError_t sm120_launch_attention_ex(const void* queries, const void* keys, const void* values, void* output,
                                      float* attention_weights, int64_t batch_size, int64_t seq_q, int64_t seq_k, int64_t head_dim,
                                      float scale, int causal, SM120DataType dtype, cudaStream_t stream) {
    if (batch_size < 0 || seq_q < 0 || seq_k < 0 || head_dim < 1) return cudaErrorInvalidValue;
    if (dtype != SM120_DTYPE_FLOAT32 && dtype != SM120_DTYPE_FLOAT16 && dtype != SM120_DTYPE_BFLOAT16)
        return cudaErrorInvalidValue;
    if (causal && seq_q > seq_k) return cudaErrorInvalidValue;
    if (batch_size == 0 || seq_q == 0) return cudaSuccess;
    if (queries == nullptr || output == nullptr || (seq_k > 0 && (keys == nullptr || values == nullptr))) return cudaErrorInvalidValue;
    if (seq_k == 0) return cudaErrorInvalidValue;                     // a softmax over no keys is undefined
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    e = query_device(device, &sms);
    if (e != cudaSuccess) return e;
    const bool fused = attention_fused_supported(dtype, batch_size, seq_q, seq_k, head_dim, queries, keys, values, output);
    // 16-bit tensors with a head dimension the fused kernel lacks have no route: the unfused one would need a
    // 16-bit [seq_q, seq_k] buffer for P that this signature does not carry
    if (!fused && dtype != SM120_DTYPE_FLOAT32) return cudaErrorInvalidValue;
    // fp32 runs unfused and needs the attention_weights buffer as its score matrix
    if (!fused && attention_weights == nullptr) return cudaErrorInvalidValue;
    if (attention_weights != nullptr) {
        // weights[b] = softmax(scale * Q[b] K[b]^T): one batched GEMM with fp32 output, then the row softmax in place
        SM120GemmDesc d;
        sm120_gemm_desc_init(&d);
        d.A = queries; d.B = keys; d.C = attention_weights;
        d.M = seq_q; d.N = seq_k; d.K = head_dim;
        d.transpose_b = 1;
        d.batch = batch_size;
        d.stride_a = seq_q * head_dim; d.stride_b = seq_k * head_dim; d.stride_c = seq_q * seq_k;
        d.in_dtype = dtype; d.out_dtype = SM120_DTYPE_FLOAT32;
        d.stream = stream;
        e = sm120_launch_matmul_ex(&d);
        if (e != cudaSuccess) return e;
        e = sm120_launch_softmax_ex(attention_weights, attention_weights, batch_size * seq_q, seq_k, SM120_DTYPE_FLOAT32,
                                    SM120_DTYPE_FLOAT32, scale, nullptr, 0, 0.0f, causal, seq_q, stream);
        if (e != cudaSuccess) return e;
    }
    if (fused) {
        e = attention_fused_launch(queries, keys, values, output, batch_size, seq_q, seq_k, head_dim, scale, causal, dtype, device,
                                   wait_limit_ns(), stream);
        if (e == cudaSuccess) {
            g_launch_count.fetch_add(1, std::memory_order_relaxed);
            t_last_kernel = head_dim == 128 ? "attention_tcgen05_d128" : "attention_tcgen05_d64";
        }
        return e;
    }
    // fp32: output[b] = weights[b] V[b]
    SM120GemmDesc d;
    sm120_gemm_desc_init(&d);
    d.A = attention_weights; d.B = values; d.C = output;
    d.M = seq_q; d.N = head_dim; d.K = seq_k;
    d.batch = batch_size;
    d.stride_a = seq_q * seq_k; d.stride_b = seq_k * head_dim; d.stride_c = seq_q * head_dim;
    d.in_dtype = dtype; d.out_dtype = dtype;
    d.stream = stream;
    return sm120_launch_matmul_ex(&d);
}

cudaError_t sm120_launch_attention(const void* queries, const void* keys, const void* values, void* output,
                                   float* attention_weights, int batch_size, int seq_len, int head_dim, float scale,
                                   SM120DataType dtype, cudaStream_t stream) {
    return sm120_launch_attention_ex(queries, keys, values, output, attention_weights, batch_size, seq_len, seq_len, head_dim, scale,
                                     0, dtype, stream);
}

bool sm120_is_supported(int device_id) {
    int sms = 0;
    return query_device(device_id, &sms) == cudaSuccess;
}

const char* sm120_get_error_string(cudaError_t error) { return cudaGetErrorString(error); }

cudaError_t sm120_get_kernel_status(int device_id, unsigned int* status, int clear) {
    if (status == nullptr) return cudaErrorInvalidValue;
    int prev = 0;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return e;
    if (prev != device_id) {
        e = cudaSetDevice(device_id);
        if (e != cudaSuccess) return e;
    }
    e = tc_read_status(status, clear);
    if (prev != device_id) cudaSetDevice(prev);
    return e;
}

void sm120_set_wait_limit_ms(unsigned int ms) {
    if (ms == 0) ms = 1;
    g_wait_limit_ns.store(static_cast<uint64_t>(ms) * 1000000ull, std::memory_order_relaxed);
}

uint64_t sm120_get_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

const char* sm120_get_last_kernel_name(void) { return t_last_kernel; }

int sm120_get_last_split_k(void) { return t_last_split_k; }

cudaError_t sm120_get_kernel_clock(int device_id, unsigned long long* cycles, unsigned long long* ns) {
    if (cycles == nullptr || ns == nullptr) return cudaErrorInvalidValue;
    int prev = 0;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return e;
    if (prev != device_id) {
        e = cudaSetDevice(device_id);
        if (e != cudaSuccess) return e;
    }
    unsigned long long both[2] = {0, 0};
    e = tc_read_probe(both);
    if (prev != device_id) cudaSetDevice(prev);
    *cycles = both[0];
    *ns = both[1];
    return e;
}

void sm120_get_tensor_map_stats(uint64_t* encoded, uint64_t* reused) {
    uint64_t e = 0, h = 0;
    tc_map_cache_stats(&e, &h);
    if (encoded != nullptr) *encoded = e;
    if (reused != nullptr) *reused = h;
}

}  // extern "C"
