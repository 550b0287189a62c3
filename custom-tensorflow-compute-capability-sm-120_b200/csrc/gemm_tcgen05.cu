// Host side of the tensor-core GEMM for B200: TMA tensor maps, tile choice,
// instruction descriptor and launch of sm120_gemm_tcgen05_kernel, whose device
// code and design notes are in gemm_tcgen05_kernel.cuh.  The kernel variants are
// instantiated in gemm_tcgen05_inst_*.cu so that they compile in parallel.
//
// Replaces the grid/dispatch part of the reference launcher
// (src/cuda_kernels/sm120_c_interface.cu:32-60) for the tensor-core path.

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>
#include <atomic>

#include "gemm_tcgen05_kernel.cuh"

namespace sm120 {

// Status and probe words of the kernel (see gemm_tcgen05_kernel.cuh), one set per device.
__device__ unsigned int g_sm120_status[4];
__device__ unsigned long long g_sm120_probe[2];

// the variants are compiled in gemm_tcgen05_inst_*.cu
#define SM120_TC_EXTERN(KIND_, BN_, ST_, CG_) \
    extern template cudaError_t launch_variant<KIND_, BN_, ST_, CG_>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const DestMaps&, \
                                                                     const TcParams&, int, int, cudaStream_t, bool);
SM120_TC_EXTERN(KIND_F16, 256, 6, 2) SM120_TC_EXTERN(KIND_F16, 256, 4, 1) SM120_TC_EXTERN(KIND_F16, 128, 6, 1) SM120_TC_EXTERN(KIND_F16, 64, 8, 1)
SM120_TC_EXTERN(KIND_F8, 256, 6, 2) SM120_TC_EXTERN(KIND_F8, 256, 4, 1) SM120_TC_EXTERN(KIND_F8, 128, 6, 1) SM120_TC_EXTERN(KIND_F8, 64, 8, 1)
SM120_TC_EXTERN(KIND_TF32, 128, 4, 2) SM120_TC_EXTERN(KIND_TF32, 128, 3, 1) SM120_TC_EXTERN(KIND_TF32, 64, 4, 1)
#undef SM120_TC_EXTERN
// the pair tile with 16 epilogue warps, for short-K (store-bound) problems
extern template cudaError_t launch_variant<KIND_F16, 256, 5, 2, 16>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const DestMaps&,
                                                                    const TcParams&, int, int, cudaStream_t, bool);
extern template cudaError_t launch_variant<KIND_F8, 256, 5, 2, 16>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const DestMaps&,
                                                                   const TcParams&, int, int, cudaStream_t, bool);

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static std::atomic<EncodeTiledFn> cached{nullptr};
    EncodeTiledFn fn = cached.load(std::memory_order_acquire);
    if (fn != nullptr) return fn;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || sym == nullptr) {
        return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(sym);
    cached.store(fn, std::memory_order_release);
    return fn;
}

static CUtensorMapDataType tmap_dtype(int dtype) {
    switch (dtype) {
        case SM120_DTYPE_FLOAT16:  return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        case SM120_DTYPE_BFLOAT16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        case SM120_DTYPE_FP8_E4M3: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
        default:                   return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    }
}

// Tensor maps are pure functions of (address, type, extents, pitches, box, swizzle), and a
// framework calls the op again and again on the same buffers and shapes, so each host thread
// keeps the maps it encoded: a direct-mapped table, thread-local and therefore free of locks
// and safe under any number of concurrent callers.  A hit costs one hash and one 64-byte
// compare instead of a driver call.
struct MapKey {
    uint64_t ptr, inner, outer, nbatch, pitch_bytes, bstride_bytes;
    uint32_t box_inner, box_outer, dtype, swizzle;
};
static_assert(sizeof(MapKey) == 64, "MapKey must have no padding: it is compared with memcmp");
struct MapSlot {
    MapKey key;
    CUtensorMap map;
    bool used;
};
constexpr int MAP_CACHE_SLOTS = 256;
static thread_local MapSlot t_map_cache[MAP_CACHE_SLOTS];
static std::atomic<uint64_t> g_map_encodes{0}, g_map_hits{0};

void tc_map_cache_stats(uint64_t* encodes, uint64_t* hits) {
    *encodes = g_map_encodes.load(std::memory_order_relaxed);
    *hits = g_map_hits.load(std::memory_order_relaxed);
}

static uint32_t map_key_hash(const MapKey& k) {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    uint64_t h = 0x9E3779B97F4A7C15ull;
    for (int i = 0; i < 8; ++i) {
        h ^= w[i];
        h *= 0xFF51AFD7ED558CCDull;
        h ^= h >> 29;
    }
    return static_cast<uint32_t>(h);
}

// 3-D map over a stored matrix: `inner` contiguous elements per row, `outer`
// rows `pitch` elements apart, `nbatch` matrices `bstride` elements apart.
static bool encode_3d(CUtensorMap* map, const void* ptr, int dtype, int64_t inner, int64_t outer, int64_t nbatch,
                      int64_t pitch, int64_t bstride, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
    const uint64_t es = static_cast<uint64_t>(dtype_size(dtype));
    MapKey key{};
    key.ptr = reinterpret_cast<uint64_t>(ptr);
    key.inner = static_cast<uint64_t>(inner); key.outer = static_cast<uint64_t>(outer); key.nbatch = static_cast<uint64_t>(nbatch);
    key.pitch_bytes = static_cast<uint64_t>(pitch) * es; key.bstride_bytes = static_cast<uint64_t>(bstride) * es;
    key.box_inner = box_inner; key.box_outer = box_outer;
    key.dtype = static_cast<uint32_t>(dtype); key.swizzle = static_cast<uint32_t>(swizzle);
    MapSlot& slot = t_map_cache[map_key_hash(key) & (MAP_CACHE_SLOTS - 1)];
    if (slot.used && memcmp(&slot.key, &key, sizeof(key)) == 0) {
        *map = slot.map;
        g_map_hits.fetch_add(1, std::memory_order_relaxed);
        return true;
    }
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[3] = {key.inner, key.outer, key.nbatch};
    cuuint64_t strides[2] = {key.pitch_bytes, key.bstride_bytes};
    cuuint32_t box[3] = {box_inner, box_outer, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, tmap_dtype(dtype), 3, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    g_map_encodes.fetch_add(1, std::memory_order_relaxed);
    slot.key = key;
    slot.map = *map;
    slot.used = true;
    return true;
}

bool tc_encode_3d(CUtensorMap* map, const void* ptr, int dtype, int64_t inner, int64_t outer, int64_t nbatch, int64_t pitch,
                  int64_t bstride, uint32_t box_inner, uint32_t box_outer) {
    return encode_3d(map, ptr, dtype, inner, outer, nbatch, pitch, bstride, box_inner, box_outer, CU_TENSOR_MAP_SWIZZLE_128B);
}

// Device address of `device`'s status words (looked up once per device, with that device current).
unsigned int* tc_status_address(int device) {
    static std::atomic<unsigned int*> status_addr[64];
    unsigned int* st = status_addr[device & 63].load(std::memory_order_acquire);
    if (st == nullptr) {
        void* a = nullptr;
        if (cudaGetSymbolAddress(&a, g_sm120_status) != cudaSuccess) return nullptr;
        st = static_cast<unsigned int*>(a);
        status_addr[device & 63].store(st, std::memory_order_release);
    }
    return st;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool tc_supported(const GemmProblem& p, const char** why) {
    auto no = [&](const char* w) { if (why) *why = w; return false; };
    if (p.in_dtype != SM120_DTYPE_FLOAT16 && p.in_dtype != SM120_DTYPE_BFLOAT16 && p.in_dtype != SM120_DTYPE_FP8_E4M3 &&
        !(p.in_dtype == SM120_DTYPE_FLOAT32 && p.tf32_operands))
        return no("input dtype has no tensor-core path");
    const int64_t es = dtype_size(p.in_dtype);
    if (p.K < 1) return no("K < 1");
    if (!aligned16(p.A) || !aligned16(p.B)) return no("A or B is not 16-byte aligned");
    if ((p.lda * es) % 16 != 0 || (p.ldb * es) % 16 != 0) return no("row pitch of A or B is not a multiple of 16 bytes");
    if (p.batch > 1) {
        if (p.stride_a != 0 && (p.stride_a * es) % 16 != 0) return no("batch stride of A is not a multiple of 16 bytes");
        if (p.stride_b != 0 && (p.stride_b * es) % 16 != 0) return no("batch stride of B is not a multiple of 16 bytes");
    }
    if (p.M >= (1ll << 31) || p.N >= (1ll << 31) || p.K >= (1ll << 31) || p.batch >= (1ll << 31)) return no("extent >= 2^31");
    const int64_t tiles = ((p.M + BM - 1) / BM) * ((p.N + 63) / 64) * p.batch;
    if (tiles >= (1ll << 31)) return no("too many tiles");
    // TMA limits: strides below 2^40 bytes
    if (p.lda * es >= (1ll << 40) || p.ldb * es >= (1ll << 40) || p.stride_a * es >= (1ll << 40) || p.stride_b * es >= (1ll << 40))
        return no("stride >= 2^40 bytes");
    return true;
}

cudaError_t tc_launch(const GemmProblem& p, uint64_t wait_limit_ns, const char** kernel_name) {
    const int es = dtype_size(p.in_dtype);
    const int epb = 128 / es;
    const int bk = epb;
    const bool fp8 = p.in_dtype == SM120_DTYPE_FP8_E4M3;
    const bool a_mn = p.transpose_a != 0;       // stored [K,M]: M contiguous
    const bool b_mn = p.transpose_b == 0;       // stored [K,N]: N contiguous

    // Tile choice.  A pair of CTAs on a 256 x 256 tile from about 25 such tiles up: the pair
    // needs half the operand bytes per MMA cycle of a 128 x 128 tile, and measured faster than
    // narrower tiles on every SM down to that size (1536^3: 36 pair tiles, 12.4 us against
    // 15.2 us; 1024^3: 16 pair tiles, 9.5 us against 6.0 us).  Otherwise the widest single-CTA
    // tile that gives every SM work; level 0 keeps
    // 128 x 128.  An MN-major operand is loaded in boxes of 128 bytes of M/N, so a
    // CTA's share of the B tile cannot be narrower than one box (128 fp8 elements).
    const int min_bn = (b_mn && es == 1) ? 128 : 64;
    // fp32 (3xTF32) tiles are at most 128 columns wide: the epilogue keeps a tile's running sums in registers
    const bool fp32 = p.in_dtype == SM120_DTYPE_FLOAT32;
    const int pair_bn = fp32 ? 128 : 256;
    auto tiles_for = [&](int bm, int bn) { return ((p.M + bm - 1) / bm) * ((p.N + bn - 1) / bn) * p.batch; };
    int cg = 1, bn = min_bn;
    // per-call overrides (SM120GemmDesc::tuning): 0 = choose, 1 / 2 = force
    const int force = (p.tuning & SM120_TUNE_CTA_GROUP_2) ? 2 : ((p.tuning & SM120_TUNE_CTA_GROUP_1) ? 1 : 0);
    if (p.optimization_level == 0) {
        bn = p.N > 64 ? 128 : min_bn;
    } else {
        if (force != 1 && p.M > 128 && p.N > pair_bn / 2 && (force == 2 || tiles_for(256, pair_bn) * 6 >= p.sm_count)) {
            cg = 2; bn = pair_bn;
        } else {
            const int wide[2] = {256, 128};
            for (int cand : wide) {
                if (cand > pair_bn) continue;
                if (p.N > cand / 2 && tiles_for(BM, cand) >= p.sm_count) { bn = cand; break; }
            }
        }
    }

    // The K parts of a split product (see splitk.cu) were counted in 128 x 128 tiles when there are at most 128 rows:
    // narrower tiles would fill the SMs on paper, but a 128 x 64 tile's MMAs are bound by shared-memory bandwidth
    // (measured on [64, 8192] x [8192, 8192]: 40 us against 31 us)
    if (p.split_k > 0 && cg == 1 && p.optimization_level != 0 && p.N > 64 && min_bn <= 128) bn = 128;
    TcParams tp{};
    tp.M = static_cast<int>(p.M); tp.N = static_cast<int>(p.N); tp.K = static_cast<int>(p.K);
    tp.batch = static_cast<int>(p.batch);
    tp.tiles_m = static_cast<int>((p.M + BM * cg - 1) / (BM * cg));
    tp.tiles_n = static_cast<int>((p.N + bn - 1) / bn);
    // fp32 path: the operands' rows are [hi | lo] (K = 2 x the padded K of the product) and a k-block of 32 feeds
    // three products.  The tensor cores' fp32 accumulation truncates, so a sum is carried in TMEM for 6 k-blocks
    // (192 elements of K) only and the runs are added in registers with round-to-nearest (see epilogue_role).
    // Measured relative Frobenius error against float64, K = 1024 and 8192 alike: 1.9e-6 on N(0,1) operands and
    // 4.3e-6 on same-sign U[0,1) operands with runs of 6; 1.2e-6 / 2.2e-6 with runs of 3 at 10 % less speed.
    tp.k_lo = fp32 ? static_cast<int>(p.K / 2) : 0;
    tp.k_blocks = static_cast<int>(((fp32 ? p.K / 2 : (p.split_k > 0 ? p.split_k : p.K)) + bk - 1) / bk);
    tp.k_split = static_cast<int>(p.split_k);
    tp.kb_per_run = fp32 ? 6 : tp.k_blocks;
    // Epilogue warps: with at most 8 k-blocks per tile the MMAs of a tile take less time than
    // its epilogue, and 16 epilogue warps (pair tiles only) hide the epilogue's latencies.
    // The same variant also serves the transcendental activations at any K: with GELU fused, 16 warps of 96
    // registers measured 5-10 % less time on the 8192 x 11008 x 4096 Dense product than 8 warps (the main
    // loop loses fewer cycles to the activation math and the SM clock settles higher under the power cap).
    const bool heavy_act = p.activation != SM120_ACTIVATION_NONE && p.activation != SM120_ACTIVATION_RELU &&
                           p.activation != SM120_ACTIVATION_LEAKY_RELU;
    int ew = (cg == 2 && p.in_dtype != SM120_DTYPE_FLOAT32 && (tp.k_blocks <= 8 || heavy_act)) ? 16 : 8;
    {
        const int fe = (p.tuning & SM120_TUNE_EPI_WARPS_16) ? 16 : ((p.tuning & SM120_TUNE_EPI_WARPS_8) ? 8 : 0);
        if (fe == 8 || (fe == 16 && cg == 2 && p.in_dtype != SM120_DTYPE_FLOAT32)) ew = fe;
    }
    tp.num_tiles = static_cast<int>(tiles_for(BM * cg, bn));
    // Raster: tiles are visited in groups of group_m row tiles, column by column, so a
    // group's slice of A (group_m x tile rows x K) stays in L2 while B streams past it once
    // per group.  The slice is sized to about a third of the 126 MB L2.
    {
        const long long slice = static_cast<long long>(BM * cg) * p.K * es;
        long long gm = (40ll << 20) / (slice > 0 ? slice : 1);
        gm = gm < 4 ? 4 : (gm > 64 ? 64 : gm);
        if (((p.tuning >> 8) & 0xFF) != 0) gm = (p.tuning >> 8) & 0xFF;
        tp.group_m = static_cast<int>(gm < tp.tiles_m ? gm : tp.tiles_m);
    }
    tp.div_per_batch = make_fast_div(static_cast<uint32_t>(tp.tiles_m) * static_cast<uint32_t>(tp.tiles_n));
    tp.div_group_span = make_fast_div(static_cast<uint32_t>(tp.group_m) * static_cast<uint32_t>(tp.tiles_n));
    tp.div_group_m = make_fast_div(static_cast<uint32_t>(tp.group_m));
    tp.div_group_last = make_fast_div(static_cast<uint32_t>(tp.tiles_m % tp.group_m == 0 ? tp.group_m : tp.tiles_m % tp.group_m));
    tp.num_work = tp.num_tiles;
    tp.full_work = tp.num_tiles;
    tp.a_mn_major = a_mn ? 1 : 0;
    tp.b_mn_major = b_mn ? 1 : 0;
    tp.a_batched = (p.batch > 1 && p.stride_a != 0 && p.split_k == 0) ? 1 : 0;
    tp.b_batched = (p.batch > 1 && p.stride_b != 0 && p.split_k == 0) ? 1 : 0;
    tp.C = p.C; tp.ldc = p.ldc; tp.stride_c = p.stride_c; tp.out_dtype = p.out_dtype;
    const int out_es = dtype_size(p.out_dtype);
    tp.c_vec_ok = (aligned16(p.C) && (p.ldc * out_es) % 16 == 0 && (p.stride_c * out_es) % 16 == 0) ? 1 : 0;
    tp.use_tma_store = (tp.c_vec_ok && p.beta == 0.0f && p.ldc * out_es < (1ll << 40) && p.stride_c * out_es < (1ll << 40)) ? 1 : 0;
    tp.bias = p.bias; tp.bias_dtype = p.bias_dtype;
    tp.bias_vec_ok = (p.bias != nullptr && aligned16(p.bias)) ? 1 : 0;
    tp.alpha = p.alpha * p.inv_scale; tp.beta = p.beta;
    tp.scale_a_dev = p.scale_a_dev; tp.scale_b_dev = p.scale_b_dev;
    tp.activation = p.activation;
    tp.stall_kblock = ((p.tuning >> 16) & 0xFF) - 1;
    tp.trace = static_cast<unsigned long long*>(p.trace);
    tp.wait_limit_ns = wait_limit_ns;
    const bool split_tail = (p.tuning & SM120_TUNE_NO_SPLIT_TAIL) == 0;
    {
        // device addresses of this device's status / probe words (looked up once per device)
        static std::atomic<unsigned long long*> probe_addr[64];
        unsigned long long* pr = probe_addr[p.device & 63].load(std::memory_order_acquire);
        if (pr == nullptr) {
            void* b = nullptr;
            if (cudaGetSymbolAddress(&b, g_sm120_probe) != cudaSuccess) return cudaErrorInvalidSymbol;
            pr = static_cast<unsigned long long*>(b);
            probe_addr[p.device & 63].store(pr, std::memory_order_release);
        }
        tp.status = tc_status_address(p.device);
        if (tp.status == nullptr) return cudaErrorInvalidSymbol;
        tp.probe = pr;
    }

    // Instruction descriptor (tcgen05.mma kind::f16 / kind::f8f6f4):
    //   bits 4..5 accumulator format (1 = f32), 7..9 A format, 10..12 B format
    //   (kind::f16: 0 = f16, 1 = bf16; kind::f8f6f4: 0 = e4m3), 15 / 16 = A / B is
    //   MN-major, 17..22 = N >> 3, 24..28 = M >> 4 (M = 256 for a CTA pair).
    const uint32_t fmt = (p.in_dtype == SM120_DTYPE_BFLOAT16) ? 1u : (p.in_dtype == SM120_DTYPE_FLOAT32 ? 2u : 0u);   // kind::tf32: 2
    tp.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(tp.a_mn_major) << 15) |
               (static_cast<uint32_t>(tp.b_mn_major) << 16) | (static_cast<uint32_t>(bn >> 3) << 17) |
               (static_cast<uint32_t>((BM * cg) >> 4) << 24);

    tp.idesc_half = (tp.idesc & ~(0x3Fu << 17)) | (static_cast<uint32_t>((bn / 2) >> 3) << 17);

    CUtensorMap ta, tb, tb_half;
    DestMaps tc;
    const int64_t nb_a = tp.a_batched ? p.batch : 1;
    const int64_t nb_b = tp.b_batched ? p.batch : 1;
    const uint32_t bn_cta = static_cast<uint32_t>(bn / cg);
    bool ok;
    if (!a_mn) ok = encode_3d(&ta, p.A, p.in_dtype, p.K, p.M, nb_a, p.lda, tp.a_batched ? p.stride_a : p.M * p.lda, bk, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    else       ok = encode_3d(&ta, p.A, p.in_dtype, p.M, p.K, nb_a, p.lda, tp.a_batched ? p.stride_a : p.K * p.lda, epb, bk, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return cudaErrorInvalidValue;
    if (!b_mn) ok = encode_3d(&tb, p.B, p.in_dtype, p.K, p.N, nb_b, p.ldb, tp.b_batched ? p.stride_b : p.N * p.ldb, bk, bn_cta, CU_TENSOR_MAP_SWIZZLE_128B);
    else       ok = encode_3d(&tb, p.B, p.in_dtype, p.N, p.K, nb_b, p.ldb, tp.b_batched ? p.stride_b : p.K * p.ldb, epb, bk, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return cudaErrorInvalidValue;
    // Half-width tiles of a short last wave (pair tiles only) load half of a CTA's share of B
    tb_half = tb;
    tp.b_bytes_half = bn_cta * 128u;
    tp.b_boxes_half = static_cast<int>(bn_cta) / epb;
    if (cg == 2) {
        if (!b_mn) {
            ok = encode_3d(&tb_half, p.B, p.in_dtype, p.K, p.N, nb_b, p.ldb, tp.b_batched ? p.stride_b : p.N * p.ldb, bk, bn_cta / 2,
                           CU_TENSOR_MAP_SWIZZLE_128B);
            if (!ok) return cudaErrorInvalidValue;
            tp.b_bytes_half = (bn_cta / 2) * 128u;
        } else if (static_cast<int>(bn_cta) / 2 >= epb) {
            tp.b_boxes_half = static_cast<int>(bn_cta) / 2 / epb;
            tp.b_bytes_half = static_cast<uint32_t>(tp.b_boxes_half) * static_cast<uint32_t>(bk) * 128u;
        }
    }
    // One TMA store writes the 32 rows of one epilogue warp x epi_cols columns: as many columns
    // as fit a 128-byte staging row, but not more than one epilogue warp owns (bn / 2, or bn / 4 with 16 warps).
    tp.epi_cols = (bn / (ew / 4) >= 64 && out_es == 2) ? 64 : 32;
    tp.epi_row_bytes = tp.epi_cols * out_es;
    tp.num_dests = 1;
    if (tp.use_tma_store) {
        const CUtensorMapSwizzle sw = tp.epi_row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
        ok = encode_3d(&tc.m[0], p.C, p.out_dtype, p.N, p.M, p.batch, p.ldc, p.batch > 1 ? p.stride_c : p.M * p.ldc,
                       static_cast<uint32_t>(tp.epi_cols), 32u, sw);
        for (int g = 0; ok && g < p.num_extra_dests; ++g) {
            ok = aligned16(p.extra_dests[g]) &&
                 encode_3d(&tc.m[1 + g], p.extra_dests[g], p.out_dtype, p.N, p.M, p.batch, p.ldc,
                           p.batch > 1 ? p.stride_c : p.M * p.ldc, static_cast<uint32_t>(tp.epi_cols), 32u, sw);
        }
        if (ok) tp.num_dests = 1 + p.num_extra_dests;
        else if (p.num_extra_dests > 0) return cudaErrorInvalidValue;
        else tp.use_tma_store = 0;
    } else if (p.num_extra_dests > 0) {
        return cudaErrorInvalidValue;        // extra destinations are written by TMA stores only
    }
    if (!tp.use_tma_store) tc.m[0] = ta;     // never dereferenced by the kernel
    tp.fast_epi = (tp.use_tma_store && p.N % 32 == 0 && (p.bias == nullptr || tp.bias_vec_ok)) ? 1 : 0;
    for (int g = tp.num_dests; g < MAX_DESTS; ++g) tc.m[g] = tc.m[0];

#define SM120_TC_CASE(KIND_, BN_, ST_, CG_, NAME_)                                                       \
    do {                                                                                                 \
        if (kernel_name) *kernel_name = NAME_;                                                           \
        return launch_variant<KIND_, BN_, ST_, CG_>(ta, tb, tb_half, tc, tp, p.sm_count, p.device, p.stream, split_tail);       \
    } while (0)

    if (p.in_dtype == SM120_DTYPE_FLOAT32) {
        // operands already split into tf32 pieces (see split_tf32.cu)
        if (cg == 2) SM120_TC_CASE(KIND_TF32, 128, 4, 2, "tc_tf32x3_2cta_256x128x32_s4");
        if (bn == 128) SM120_TC_CASE(KIND_TF32, 128, 3, 1, "tc_tf32x3_128x128x32_s3");
        SM120_TC_CASE(KIND_TF32, 64, 4, 1, "tc_tf32x3_128x64x32_s4");
    } else if (!fp8) {
        const bool bf = p.in_dtype == SM120_DTYPE_BFLOAT16;
        if (cg == 2 && ew == 16) {
            if (kernel_name) *kernel_name = bf ? "tc_bf16_2cta_256x256x64_s5_e16" : "tc_f16_2cta_256x256x64_s5_e16";
            return launch_variant<KIND_F16, 256, 5, 2, 16>(ta, tb, tb_half, tc, tp, p.sm_count, p.device, p.stream, split_tail);
        }
        if (cg == 2) SM120_TC_CASE(KIND_F16, 256, 6, 2, bf ? "tc_bf16_2cta_256x256x64_s6" : "tc_f16_2cta_256x256x64_s6");
        if (bn == 256) SM120_TC_CASE(KIND_F16, 256, 4, 1, bf ? "tc_bf16_128x256x64_s4" : "tc_f16_128x256x64_s4");
        if (bn == 128) SM120_TC_CASE(KIND_F16, 128, 6, 1, bf ? "tc_bf16_128x128x64_s6" : "tc_f16_128x128x64_s6");
        SM120_TC_CASE(KIND_F16, 64, 8, 1, bf ? "tc_bf16_128x64x64_s8" : "tc_f16_128x64x64_s8");
    } else {
        if (cg == 2 && ew == 16) {
            if (kernel_name) *kernel_name = "tc_e4m3_2cta_256x256x128_s5_e16";
            return launch_variant<KIND_F8, 256, 5, 2, 16>(ta, tb, tb_half, tc, tp, p.sm_count, p.device, p.stream, split_tail);
        }
        if (cg == 2) SM120_TC_CASE(KIND_F8, 256, 6, 2, "tc_e4m3_2cta_256x256x128_s6");
        if (bn == 256) SM120_TC_CASE(KIND_F8, 256, 4, 1, "tc_e4m3_128x256x128_s4");
        if (bn == 128) SM120_TC_CASE(KIND_F8, 128, 6, 1, "tc_e4m3_128x128x128_s6");
        SM120_TC_CASE(KIND_F8, 64, 8, 1, "tc_e4m3_128x64x128_s8");
    }
#undef SM120_TC_CASE
}

cudaError_t tc_read_probe(unsigned long long* cycles_ns) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    return cudaMemcpyFromSymbol(cycles_ns, g_sm120_probe, 2 * sizeof(unsigned long long));
}

cudaError_t tc_read_status(unsigned int* status, int clear) {
    unsigned int host[4] = {0, 0, 0, 0};
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    e = cudaMemcpyFromSymbol(host, g_sm120_status, sizeof(host));
    if (e != cudaSuccess) return e;
    if (status) { status[0] = host[0]; }
    if (clear && (host[0] != 0 || host[1] != 0)) {
        unsigned int zero[4] = {0, 0, 0, 0};
        e = cudaMemcpyToSymbol(g_sm120_status, zero, sizeof(zero));
    }
    return e;
}

}  // namespace sm120
