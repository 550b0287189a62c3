#pragma once
// Tensor-core GEMM for B200 (sm_100a): tcgen05.mma with fp32 accumulators in
// tensor memory (TMEM), operands staged in shared memory by TMA through a
// multi-stage mbarrier ring, warp-specialised roles, persistent CTAs, and an
// epilogue that goes TMEM -> registers -> swizzled shared memory -> TMA store.
//
// It replaces the reference's WMMA-tiled GEMM family
// (src/cuda_kernels/sm120_optimized_kernels_fixed.cu:133-286 and :458-509) and
// the naive kernel behind its C launcher
// (src/cuda_kernels/sm120_pure_kernels.cu:19-65), and adds the strided-batch
// form of src/cuda_kernels/sm120_dynamic_shapes.cu:107-183 and the fused
// bias + activation + cast epilogue.
//
// One CTA = 2 + EW warps (EW = 8, or 16 for short-K problems):
//   warp 0      TMA producer (one elected lane issues): fills the shared-memory ring
//   warp 1      TMEM allocator; one elected lane issues tcgen05.mma and the commits
//   warps 2..   epilogue.  Warp w reads TMEM lanes [32*(w%4), +32) (the hardware
//               ties a warp to that quarter) and the column part (w-2)/4 of the
//               tile (a half with 8 warps, a quarter with 16), 32 columns at a time:
//               tcgen05.ld, alpha/scale, bias, activation, cast, swizzled st.shared
//               into the warp's own staging buffer, and one TMA store per
//               32 rows x 64 (or 32) columns.  Epilogue warps never wait for one another.
//
// Two flavours, chosen by the template parameter CG:
//   CG = 1  one CTA per tile of 128 x BN (BN = 64, 128, 256).
//   CG = 2  a cluster of two CTAs per tile of 256 x 256 (tcgen05 cta_group::2).
//           CTA r of the pair loads rows [128r, 128r+128) of the A tile and columns
//           [128r, 128r+128) of the B tile into its own shared memory; the MMA
//           issued by CTA 0 reads both CTAs' shared memory and writes both CTAs'
//           TMEM (each CTA ends up with its 128 rows x 256 columns).  Per CTA this
//           moves 32 KB per k-block from L2 instead of 48 KB for the same math.
//           The TMA loads use no cluster multicast.
// The accumulator is double buffered in TMEM, so the epilogue of one tile overlaps
// the main loop of the next.  Tiles are handed out statically; there is no
// split-K and no atomic, so results are bitwise reproducible from run to run.
//
// Operand layouts.  Each operand tile in shared memory is a sequence of
// 128-byte-swizzled atoms exactly as TMA writes them:
//   K-major operand (K contiguous in memory: A not transposed, B transposed):
//     one box {BK, rows}: row r at r*128 B, 8-row groups 1024 B apart.
//   MN-major operand (M or N contiguous: A transposed, B not transposed):
//     rows*es/128 boxes {128/es, BK}: box j covers 128 bytes of M/N; inside a box
//     k-row k is at k*128 B.
// BK is always 128 bytes of K (64 bf16/fp16, 128 fp8), i.e. 4 MMA K-steps of 32 B.
//
// Every wait on an mbarrier is bounded by a wall-clock limit.  A role whose
// wait runs out records a code in the status words, raises the CTA's abort flag
// (and its peer's) and leaves; the other roles see the flag in their own wait
// loops; the CTA then waits (bounded) for its TMA copies and MMAs in flight,
// frees its TMEM and returns normally.

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>

#include "gemm_common.h"

namespace sm120 {

// The kernel reports through two small device arrays that the host side owns
// (TcParams::status, TcParams::probe):
//   status[0]: first timeout code seen (role<<28 | barrier kind<<24 | CTA), status[1]: number of waits that ran out;
//   probe[0] / probe[1]: SM cycles and nanoseconds that CTA 0 of the last launch was alive (clock probe for tuning).

enum : int { KIND_F16 = 0, KIND_F8 = 1, KIND_TF32 = 2 };
enum : int { ACTC_NONE = 0, ACTC_RELU = 1, ACTC_GELU_ERF = 2, ACTC_DYNAMIC = 3 };

constexpr int BM = 128;                 // rows per CTA
// Epilogue warps per CTA (template parameter EW): 8 split a tile's columns in two halves, 16 in four
// quarters (twice the warps to hide the latencies of a store-bound, short-K problem; 96 registers each).
constexpr uint32_t EPI_STAGE_BYTES = 4096;   // one staging buffer of an epilogue warp: 32 rows x 128 B

constexpr int EPI_PREFETCH = 2;             // 32-column TMEM loads an epilogue warp keeps in flight
constexpr int MAX_DESTS = 8;
// Tensor maps of the output: entry 0 is the caller's C; entries 1.. are further
// copies of the same [M, N] block in other buffers (other GPUs' memory when the
// launch also performs the all-gather of an M-sharded product).
struct DestMaps { CUtensorMap m[MAX_DESTS]; };

// Optional timeline of a launch (TcParams::trace, null in normal launches): every CTA owns
// TRACE_WORDS 64-bit words of a caller-provided buffer; the layout is documented with
// SM120_TUNE_TRACE in the public header.
constexpr int TRACE_WORDS = SM120_TRACE_WORDS_PER_CTA;
constexpr int TRACE_TILES = 8;

// Division by a value fixed at launch: q = (umulhi(n, mul) + n) >> shift for 0 <= n < 2^31.
struct FastDiv {
    uint32_t div, mul, shift;
};
inline FastDiv make_fast_div(uint32_t d) {
    FastDiv f{d, 1u, 0u};
    if (d <= 1u) { f.div = 1u; return f; }
    uint32_t s = 0;
    while ((1ull << s) < d) ++s;
    f.shift = s;
    f.mul = static_cast<uint32_t>(((1ull << 32) * ((1ull << s) - d)) / d + 1ull);
    return f;
}
__device__ __forceinline__ int fast_div(int n, const FastDiv& f) {
    return static_cast<int>((__umulhi(static_cast<uint32_t>(n), f.mul) + static_cast<uint32_t>(n)) >> f.shift);
}

struct TcParams {
    int M, N, K, batch;
    int tiles_m, tiles_n, k_blocks, num_tiles;   // tiles are (CG*128) x BN
    int kb_per_run;                 // k-blocks summed in TMEM before the epilogue takes the partial sum (k_blocks: one run per tile)
    int k_lo;                       // fp32 path: K coordinate at which the operands' low pieces start (their rows are [hi | lo])
    int k_split;                    // split-K: batch entry z covers K coordinates [z * k_split, (z + 1) * k_split) of unbatched operands; else 0
    int group_m;                    // row tiles per raster group (tiles of a group share their B columns in L2)
    FastDiv div_per_batch;          // tiles_m * tiles_n
    FastDiv div_group_span;         // group_m * tiles_n
    FastDiv div_group_m;            // rows of a whole group
    FastDiv div_group_last;         // rows of the last (possibly shorter) group
    int num_work, full_work;        // work items: [0, full_work) are whole tiles, the rest are half-width tiles (two per tile)
    uint32_t idesc;
    uint32_t idesc_half;            // instruction descriptor of a half-width tile (N = BN / 2)
    uint32_t b_bytes_half;          // bytes of B one CTA loads per k-block of a half-width tile
    int b_boxes_half;               // MN-major B: 128-byte boxes of N per CTA in a half-width tile
    int a_mn_major, b_mn_major;
    int a_batched, b_batched;
    void* C;
    long long ldc, stride_c;
    int out_dtype;
    int c_vec_ok;                   // C rows may be written with 16-byte stores
    int use_tma_store;              // epilogue goes through shared memory and TMA (needs beta == 0, aligned C)
    int fast_epi;                   // use_tma_store, N % 32 == 0 and a bias (if any) that 16-byte loads can read: straight-line epilogue
    int num_dests;                  // how many of DestMaps::m every output block is stored to (>= 1)
    int epi_cols;                   // columns per TMA store: 64 or 32 (one staging row of 128 or 64 bytes)
    int epi_row_bytes;              // bytes per staging row: 128 or 64
    const void* bias;
    int bias_dtype;
    int bias_vec_ok;                // bias is 16-byte aligned
    float alpha, beta;
    const float* scale_a_dev;
    const float* scale_b_dev;
    int activation;
    int stall_kblock;               // >= 0: the producer never fills this k-block of its first tile (self-test of the bounded waits)
    unsigned long long wait_limit_ns;
    unsigned int* status;           // device array of 4 words, see above
    unsigned long long* probe;      // device array of 2 words, see above
    unsigned long long* trace;      // null, or the caller's timeline buffer (see TRACE_WORDS)
};

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
// true in exactly one lane of a fully active warp
__device__ __forceinline__ bool elect_one_sync() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xFFFFFFFF;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrive on a barrier given by a shared::cluster address (own or peer CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t holder_smem, uint32_t ncols) {
    if constexpr (CG == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(ncols) : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(ncols) : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (CG == 1)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    if constexpr (CG == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive on the mbarrier at shared::cluster address `bar` once every tcgen05.mma
// issued so far by this thread has retired.
template <int CG>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    if constexpr (CG == 1)
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Tiled TMA load of one 3-D box into this CTA's shared memory; completion is
// signalled as transaction bytes on `bar`.  With CG == 2 `bar` may be the
// shared::cluster address of the pair leader's barrier.  No cluster multicast.
template <int CG>
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint32_t bar, int x, int y, int z) {
    if constexpr (CG == 1)
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z)
            : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z)
            : "memory");
}
// Tiled TMA store of one 3-D box from shared memory; out-of-range rows and
// columns of the box are clipped by the hardware.
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int KIND, int CG>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (KIND == KIND_F16 && CG == 1) {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    } else if constexpr (KIND == KIND_F16 && CG == 2) {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    } else if constexpr (KIND == KIND_TF32 && CG == 1) {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    } else if constexpr (KIND == KIND_TF32 && CG == 2) {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    } else if constexpr (KIND == KIND_F8 && CG == 1) {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    }
}

// 32 TMEM lanes x 32 consecutive 32-bit columns -> 32 registers per thread
// (thread i of the warp owns lane i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
// The same load and the wait for it in one statement: the registers are valid when it returns.
// (With the split form the compiler may copy or spill the destination registers between the load
// and the wait, while the hardware has not written them yet; that is only safe where register
// pressure is low.)
__device__ __forceinline__ void tmem_ld_32x32_sync(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (tcgen05 form, version 1, 128-byte swizzle):
//   bits  0..13  start address >> 4
//   bits 16..29  leading-dimension byte offset >> 4
//   bits 32..45  stride-dimension byte offset >> 4
//   bits 46..47  descriptor version (1 on sm_100)
//   bits 61..63  layout type (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFF);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// ---------------------------------------------------------------------------
// Bounded wait.  `code` identifies role and barrier for the status word.
// ---------------------------------------------------------------------------
struct WaitCtx {
    unsigned int* status;               // device status words
    volatile uint32_t* abort_flag;      // this CTA's flag
    uint32_t peer_abort_addr;           // shared::cluster address of the peer CTA's flag, 0 without a peer
    unsigned long long limit_ns;
};

__device__ __forceinline__ void raise_abort(const WaitCtx& w, uint32_t code) {
    *w.abort_flag = 1u;
    if (w.peer_abort_addr != 0u)
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(w.peer_abort_addr), "r"(1u) : "memory");
    atomicCAS(&w.status[0], 0u, code | (blockIdx.x & 0xFFFFFFu));
    atomicAdd(&w.status[1], 1u);
}

static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, const WaitCtx& w, uint32_t code, bool watch_abort) {
    const unsigned long long t0 = global_timer_ns();
    uint32_t spins = 0;
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 31u) == 0u) {
            if (watch_abort && *w.abort_flag != 0u) return false;
            if (global_timer_ns() - t0 > w.limit_ns) {
                raise_abort(w, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w, uint32_t code, bool watch_abort = true) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, w, code, watch_abort);
}

__device__ __forceinline__ void decode_tile(int tile, const TcParams& p, int& bz, int& tm, int& tn) {
    bz = fast_div(tile, p.div_per_batch);
    const int t = tile - bz * static_cast<int>(p.div_per_batch.div);
    const int g = fast_div(t, p.div_group_span);
    const int first_m = g * p.group_m;
    const int r = t - g * static_cast<int>(p.div_group_span.div);
    const bool last = first_m + p.group_m > p.tiles_m;          // the shorter group at the bottom
    const int gm = last ? static_cast<int>(p.div_group_last.div) : p.group_m;
    tn = last ? fast_div(r, p.div_group_last) : fast_div(r, p.div_group_m);
    tm = first_m + (r - tn * gm);
}

// Work item -> batch entry, row tile, first column and width.  The last
// num_work - full_work items are the two column halves of the last tiles: when the
// tile count leaves the final wave less than half full, splitting those tiles
// shortens the tail from one tile time to half a tile time.
__device__ __forceinline__ void decode_work(int w, const TcParams& p, int bn, int& bz, int& tm, int& n0, int& width) {
    int tile = w, sel = 0;
    width = bn;
    if (w >= p.full_work) {
        const int h = w - p.full_work;
        tile = p.full_work + (h >> 1);
        sel = h & 1;
        width = bn >> 1;
    }
    int tn;
    decode_tile(tile, p, bz, tm, tn);
    n0 = tn * bn + sel * width;
}

// ---------------------------------------------------------------------------
// Epilogue helpers.  Everything is fully unrolled over compile-time indices so
// that the 32 values of a row segment stay in registers.
// ---------------------------------------------------------------------------
// GELU with the exact (erf) definition, evaluated with the Abramowitz-Stegun
// 7.1.26 rational approximation of erf (|error| <= 1.5e-7) and the hardware
// exponential: about a third of the instructions of erff().  Measured against
// the float64 definition the absolute error of the result stays below 5e-7.
__device__ __forceinline__ float gelu_erf_fast(float x) {
    const float z = x * 0.70710678118654752440f;
    const float az = fabsf(z);
    const float t = __fdividef(1.0f, fmaf(0.3275911f, az, 1.0f));
    float poly = 1.061405429f;
    poly = fmaf(poly, t, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    poly *= t;
    const float erf_abs = fmaf(-poly, __expf(-az * az), 1.0f);
    return 0.5f * x * (1.0f + copysignf(erf_abs, z));
}

// The same for two values at once on sm_100's packed fp32 arithmetic (fma.rn.f32x2 and friends: one issue slot for
// two results).  In the fused Dense epilogue the activation competes with the tensor pipe's feed for issue slots;
// the polynomial, the products and the final scaling take half as many this way.  Same formula, same constants.
__device__ __forceinline__ uint64_t epi_pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void epi_split2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t epi_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t epi_mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ void gelu_erf_fast2(float& x0, float& x1) {
    const uint64_t x2 = epi_pack2(x0, x1);
    float z0, z1;
    epi_split2(epi_mul2(x2, epi_pack2(0.70710678118654752440f, 0.70710678118654752440f)), z0, z1);
    const uint64_t az2 = epi_pack2(fabsf(z0), fabsf(z1));
    float d0, d1;
    epi_split2(epi_fma2(az2, epi_pack2(0.3275911f, 0.3275911f), epi_pack2(1.0f, 1.0f)), d0, d1);
    const uint64_t t2 = epi_pack2(__fdividef(1.0f, d0), __fdividef(1.0f, d1));
    uint64_t poly = epi_fma2(epi_pack2(1.061405429f, 1.061405429f), t2, epi_pack2(-1.453152027f, -1.453152027f));
    poly = epi_fma2(poly, t2, epi_pack2(1.421413741f, 1.421413741f));
    poly = epi_fma2(poly, t2, epi_pack2(-0.284496736f, -0.284496736f));
    poly = epi_fma2(poly, t2, epi_pack2(0.254829592f, 0.254829592f));
    poly = epi_mul2(poly, t2);
    float s0, s1;
    epi_split2(epi_mul2(az2, az2), s0, s1);
    const uint64_t e2 = epi_pack2(__expf(-s0), __expf(-s1));
    float a0, a1;
    epi_split2(epi_fma2(epi_mul2(poly, e2), epi_pack2(-1.0f, -1.0f), epi_pack2(1.0f, 1.0f)), a0, a1);      // |erf|
    const uint64_t one_plus = epi_pack2(1.0f + copysignf(a0, z0), 1.0f + copysignf(a1, z1));
    epi_split2(epi_mul2(epi_mul2(x2, epi_pack2(0.5f, 0.5f)), one_plus), x0, x1);
}

template <int ACT>
__device__ __forceinline__ void act_loop(float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = apply_activation(v[j], ACT);     // ACT is a constant: the switch folds
}

// Apply the activation to the 32 values.  The three common cases are compile-time
// (ACTC); the rest dispatch ONCE per 32 values so that only one formula's code is
// executed (a switch inside the unrolled loop would put every formula 32 times
// into the instruction stream).
template <int ACTC>
__device__ __forceinline__ void act_apply32(float (&v)[32], int act) {
    if constexpr (ACTC == ACTC_NONE) {
        return;
    } else if constexpr (ACTC == ACTC_RELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = fmaxf(0.0f, v[j]);
    } else if constexpr (ACTC == ACTC_GELU_ERF) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) gelu_erf_fast2(v[j], v[j + 1]);
    } else {
        switch (act) {
            case SM120_ACTIVATION_RELU:       act_apply32<ACTC_RELU>(v, act); break;
            case SM120_ACTIVATION_GELU_ERF:   act_apply32<ACTC_GELU_ERF>(v, act); break;
            case SM120_ACTIVATION_LEAKY_RELU: act_loop<SM120_ACTIVATION_LEAKY_RELU>(v); break;
            case SM120_ACTIVATION_ELU:        act_loop<SM120_ACTIVATION_ELU>(v); break;
            case SM120_ACTIVATION_SELU:       act_loop<SM120_ACTIVATION_SELU>(v); break;
            case SM120_ACTIVATION_GELU:       act_loop<SM120_ACTIVATION_GELU>(v); break;
            case SM120_ACTIVATION_SWISH:      act_loop<SM120_ACTIVATION_SWISH>(v); break;
            case SM120_ACTIVATION_MISH:       act_loop<SM120_ACTIVATION_MISH>(v); break;
            case SM120_ACTIVATION_TANH:       act_loop<SM120_ACTIVATION_TANH>(v); break;
            case SM120_ACTIVATION_SIGMOID:    act_loop<SM120_ACTIVATION_SIGMOID>(v); break;
            default: break;
        }
    }
}

// Bias for 32 consecutive columns.  A 16-bit bias (64 bytes) is fetched early as
// four raw 16-byte words (every lane reads the same addresses) and added later,
// so that the load latency overlaps other work; an fp32 bias is read where it is
// added (prefetching its 32 registers would spill).
struct BiasRaw { uint4 q[4]; };

__device__ __forceinline__ void bias_prefetch32(const TcParams& p, int col0, BiasRaw& r) {
    if (p.bias_dtype != SM120_DTYPE_FLOAT32) {
        const uint4* b = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.bias) + col0);
#pragma unroll
        for (int j = 0; j < 4; ++j) r.q[j] = __ldg(b + j);
    }
}

__device__ __forceinline__ void bias_add_raw32(const TcParams& p, int col0, const BiasRaw& r, float (&v)[32]) {
    if (p.bias_dtype == SM120_DTYPE_FLOAT32) {
        const float4* b4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.bias) + col0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 b = __ldg(b4 + j);
            v[4 * j + 0] += b.x; v[4 * j + 1] += b.y; v[4 * j + 2] += b.z; v[4 * j + 3] += b.w;
        }
    } else {
        const bool is_bf16 = p.bias_dtype == SM120_DTYPE_BFLOAT16;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t w[4] = {r.q[j].x, r.q[j].y, r.q[j].z, r.q[j].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float lo, hi;
                if (is_bf16) {
                    lo = __uint_as_float(w[k] << 16);
                    hi = __uint_as_float(w[k] & 0xFFFF0000u);
                } else {
                    const __half2 h = *reinterpret_cast<const __half2*>(&w[k]);
                    lo = __low2float(h);
                    hi = __high2float(h);
                }
                v[8 * j + 2 * k] += lo;
                v[8 * j + 2 * k + 1] += hi;
            }
        }
    }
}

// v[j] += bias[col0 + j] for j < ncols, element by element (ragged or unaligned bias)
__device__ __forceinline__ void bias_add_scalar32(const TcParams& p, int col0, int ncols, float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
        if (j < ncols) v[j] += load_as_float(p.bias, col0 + j, p.bias_dtype);
}

// tcgen05.wait::ld that also names the destination registers of the load, so
// that no use of them can be scheduled ahead of the wait.
__device__ __forceinline__ void tmem_ld_wait_regs(uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;"
        : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
          "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
          "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
          "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
        :
        : "memory");
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ void pack16(const float (&v)[32], bool bf16, uint32_t (&packed)[16]) {
    if (bf16) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            packed[j] = *reinterpret_cast<uint32_t*>(&h);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
            packed[j] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
}

// Write this thread's 32 values into row `r` (0..127) of the staging block of its
// column half, laid out as the TMA store expects it.  Rows are `row_bytes` long
// (128 or 64); the 32 values fill 16-byte chunks [first_chunk, first_chunk + n)
// of the row (n = 8 for fp32, 4 for 16-bit types); chunk c of row r is stored at
// chunk c ^ (r & 7) under the 128-byte swizzle and at c ^ ((r >> 1) & 3) under the
// 64-byte swizzle, which also keeps the st.shared free of bank conflicts.
__device__ __forceinline__ void stage_row32(uint32_t block_addr, int r, int row_bytes, int first_chunk,
                                            const float (&v)[32], int out_dtype) {
    const uint32_t row = block_addr + r * row_bytes;
    const int sw = (row_bytes == 128) ? (r & 7) : ((r >> 1) & 3);
    if (out_dtype == SM120_DTYPE_FLOAT32) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
            st_shared_v4(row + (((first_chunk + c) ^ sw) << 4), __float_as_uint(v[4 * c]), __float_as_uint(v[4 * c + 1]),
                         __float_as_uint(v[4 * c + 2]), __float_as_uint(v[4 * c + 3]));
    } else {
        uint32_t packed[16];
        pack16(v, out_dtype == SM120_DTYPE_BFLOAT16, packed);
#pragma unroll
        for (int c = 0; c < 4; ++c)
            st_shared_v4(row + (((first_chunk + c) ^ sw) << 4), packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
    }
}

// Direct path: this lane writes its row segment to global memory itself (used
// when beta != 0 or when C cannot be described to TMA).
__device__ __forceinline__ void store_row32_direct(const TcParams& p, long long off, int ncols, const float (&v)[32]) {
    if (ncols == 32 && p.c_vec_ok) {
        if (p.out_dtype == SM120_DTYPE_FLOAT32) {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.C) + off);
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
            uint32_t packed[16];
            pack16(v, p.out_dtype == SM120_DTYPE_BFLOAT16, packed);
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.C) + off);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < ncols) store_from_float(p.C, off + j, p.out_dtype, v[j]);
    }
}

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
template <int KIND, int BN, int STAGES, int CG, int EW = 8>
struct TileCfg {
    static constexpr int THREADS = 64 + 32 * EW;
    static constexpr int NSPLIT = EW / 4;           // column parts of a tile, one per group of four epilogue warps
    static constexpr int ES = (KIND == KIND_F16) ? 2 : (KIND == KIND_F8 ? 1 : 4);
    static constexpr int EPB = 128 / ES;            // elements per 128 bytes
    static constexpr int BK = EPB;                  // K elements per stage
    static constexpr int UMMA_K = 32 / ES;          // K elements per tcgen05.mma
    static constexpr int BN_CTA = BN / CG;          // columns of the B tile this CTA loads
    static constexpr uint32_t A_BYTES = BM * 128;
    static constexpr uint32_t B_BYTES = BN_CTA * 128;
    static constexpr uint32_t PAIR_BYTES = A_BYTES + B_BYTES;     // one A tile and one B tile
    // fp32 path (3xTF32): a stage holds the high AND the low pieces of both operands, [A_hi][B_hi][A_lo][B_lo], and
    // feeds three products (hi.hi, hi.lo, lo.hi): 1.5x less shared-memory fill per product than a stage per product
    static constexpr int PARTS = (KIND == KIND_TF32) ? 2 : 1;
    static constexpr uint32_t STAGE_BYTES = PARTS * PAIR_BYTES;
    static constexpr uint32_t MN_BOX_BYTES = BK * 128;   // one {128 B of M/N, BK} box
    static constexpr uint32_t TMEM_COLS = 2 * BN;        // 128, 256 or 512: a power of two >= 32
    static constexpr uint32_t BAR_BYTES = 256;
    // two staging buffers per epilogue warp where the pipeline stages leave room, else one
    static constexpr int EPI_BUFS =
        (size_t(STAGES) * STAGE_BYTES + 2 * EW * EPI_STAGE_BYTES + BAR_BYTES + 1024 <= 232448) ? 2 : 1;
    static constexpr uint32_t EPI_BYTES = EW * EPI_BUFS * EPI_STAGE_BYTES;
    static_assert(EW == 8 || EW == 16, "epilogue warps");
    static_assert(BN >= 32 * NSPLIT, "every epilogue warp needs at least 32 columns");
    static constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024 /* alignment slack */;
    static_assert(BN_CTA % 64 == 0 && BN % 64 == 0, "tile width");
    static_assert((2 * STAGES + 5) * 8 + 8 <= BAR_BYTES, "barrier block");
    static_assert(SMEM <= 232448, "shared memory budget exceeded");
    static_assert(SMEM > 116224, "one CTA per SM is assumed: shared memory must exceed half of an SM's");
};

// General epilogue: any N, beta, output alignment; and the run-wise accumulation of the fp32
// (3xTF32) path.  There a tile's K range is cut into runs of TcParams::kb_per_run k-blocks; the
// tensor cores sum one run in TMEM (their fp32 accumulation truncates, so the error of a run grows
// with its length), this role adds the runs in registers with round-to-nearest fp32 adds, and
// the two TMEM buffers alternate between runs so the adds overlap the next run's MMAs.
template <int KIND, int BN, int STAGES, int CG, int EW, int ACTC>
__device__ __forceinline__ void epilogue_role(const TcParams& p, const DestMaps* dests, const WaitCtx& wctx,
                                              uint32_t tmem_base, uint32_t acc_full_bar, uint32_t acc_empty_addr,
                                              uint32_t stage_addr, int warp, int lane, uint32_t cta_rank, int first_tile,
                                              int tile_step) {
    constexpr int EPI_BUFS = TileCfg<KIND, BN, STAGES, CG, EW>::EPI_BUFS;
    constexpr int NSPLIT = EW / 4;
    constexpr bool RUNS = KIND == KIND_TF32;  // several accumulation runs per tile, summed here
    const int lane_group = warp & 3;          // TMEM lanes [32*lane_group, +32) belong to this warp
    const int half = (warp - 2) >> 2;         // which part (half or quarter) of the tile's columns
    constexpr int CHUNKS = BN / (32 * NSPLIT); // 32-column chunks per warp in a whole tile
    static_assert(!RUNS || CHUNKS <= 2, "the run sums of the fp32 path live in registers: at most 64 columns per thread");
    float alpha = p.alpha;
    if (p.scale_a_dev != nullptr) alpha /= __ldg(p.scale_a_dev);
    if (p.scale_b_dev != nullptr) alpha /= __ldg(p.scale_b_dev);
    const bool has_bias = p.bias != nullptr;
    const int spg = p.epi_cols >> 5;                    // 32-column chunks per TMA store: 1 or 2
    const int chunk16_per_sub = (p.out_dtype == SM120_DTYPE_FLOAT32) ? 8 : 4;
    uint32_t stores = 0;                                // TMA stores committed by this warp: picks the staging buffer
    uint32_t acc_iter = 0;                              // accumulation runs consumed so far: picks the TMEM buffer and the phase
    for (int tile = first_tile; tile < p.num_work; tile += tile_step) {
        int bz, tm, n0, width;
        decode_work(tile, p, BN, bz, tm, n0, width);
        const int row0 = (tm * CG + static_cast<int>(cta_rank)) * BM + lane_group * 32;   // first row of this warp
        const int row = row0 + lane;
        const int cols_per_warp = width / NSPLIT;
        const int colbase = n0 + half * cols_per_warp;
        // chunks of 32 columns this warp owns that start inside the matrix (warp-uniform)
        const int nvalid = max(0, min(cols_per_warp >> 5, (p.N - colbase + 31) / 32));
        BiasRaw braw;
        // the first chunk's bias is fetched before the wait for the accumulator
        if (has_bias && p.bias_vec_ok && nvalid > 0 && colbase + 32 <= p.N) bias_prefetch32(p, colbase, braw);

        constexpr int SUMC = RUNS ? CHUNKS : 1;
        float sum[SUMC][32];
        uint32_t buf = acc_iter & 1u;
        if constexpr (RUNS) {
            bool ok = true;
            for (int kb0 = 0; kb0 < p.k_blocks; kb0 += p.kb_per_run, ++acc_iter) {
                buf = acc_iter & 1u;
                ok = mbar_wait(acc_full_bar + 8 * buf, (acc_iter >> 1) & 1u, wctx, 0x31000000u);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t t_run = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + buf * BN + half * cols_per_warp;
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) {
                    if (c < nvalid) {
                        uint32_t part[32];
                        __syncwarp();
                        tmem_ld_32x32_sync(t_run + c * 32, part);
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            sum[c][j] = (kb0 == 0) ? __uint_as_float(part[j]) : __fadd_rn(sum[c][j], __uint_as_float(part[j]));
                    }
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acc_empty_addr + 8 * buf);
            }
            if (!ok) break;
        } else {
            bool ok = mbar_wait(acc_full_bar + 8 * buf, (acc_iter >> 1) & 1u, wctx, 0x31000000u);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            ++acc_iter;
        }
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + buf * BN + half * cols_per_warp;

        // (this path is register-heavy: every TMEM load and its wait are one step)
        uint32_t acc[1][32];
        constexpr int MODP = 1;
        constexpr int PRE = 0;
        __syncwarp();
        if (!RUNS && nvalid == 0) {
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_addr + 8 * buf);
        }

#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            if (c < nvalid) {                               // warp-uniform
                const int col0 = colbase + c * 32;
                const int ncols = min(32, p.N - col0);
                if constexpr (!RUNS) {
                    __syncwarp();
                    tmem_ld_32x32_sync(t_row + c * 32, acc[0]);
                    if (c == nvalid - 1) {                  // nothing more to load: hand the TMEM buffer back
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(acc_empty_addr + 8 * buf);
                    }
                }
                float v[32];
                if constexpr (RUNS) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = alpha * sum[c < SUMC ? c : 0][j];
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = alpha * __uint_as_float(acc[c % MODP][j]);
                }
                (void)PRE;
                const long long off = static_cast<long long>(bz) * p.stride_c + static_cast<long long>(row) * p.ldc + col0;
                if (p.beta != 0.0f && row < p.M) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (j < ncols) v[j] += p.beta * load_as_float(p.C, off + j, p.out_dtype);
                }
                if (has_bias) {
                    if (p.bias_vec_ok && ncols == 32) bias_add_raw32(p, col0, braw, v);
                    else bias_add_scalar32(p, col0, ncols, v);
                    // fetch the next chunk's bias now; it is consumed one chunk later
                    if (p.bias_vec_ok && c + 1 < nvalid && col0 + 64 <= p.N) bias_prefetch32(p, col0 + 32, braw);
                }
                act_apply32<ACTC>(v, p.activation);

                if (p.use_tma_store) {
                    // Each warp stages and stores its own 32 rows: no barrier with the other warps.
                    const int sub = (spg == 2) ? (c & 1) : 0;           // position of this chunk in its store
                    const bool first_of_store = sub == 0;
                    const bool last_of_store = (sub == spg - 1) || (c == nvalid - 1);
                    const uint32_t sbuf = stage_addr + (EPI_BUFS == 2 ? (stores & 1u) * EPI_STAGE_BYTES : 0u);
                    if (first_of_store) {
                        // the staging buffer is about to be overwritten: the TMA store that last used it must have read it
                        if (lane == 0) bulk_wait_group_read<EPI_BUFS - 1>();
                        __syncwarp();
                    }
                    stage_row32(sbuf, lane, p.epi_row_bytes, sub * chunk16_per_sub, v, p.out_dtype);
                    if (last_of_store) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            if (row0 < p.M) {
                                for (int g = 0; g < p.num_dests; ++g)      // own C, then every peer's copy
                                    tma_store_3d(&dests->m[g], sbuf, col0 - sub * 32, row0, bz);
                            }
                            bulk_commit_group();
                        }
                        ++stores;
                    }
                } else if (row < p.M) {
                    store_row32_direct(p, off, ncols, v);
                }
            }
        }
    }
    if (lane == 0) {
        bulk_wait_group_read<0>();     // shared memory must outlive the stores that read it
        if (p.num_dests > 1) {
            // copies that went to other GPUs: wait for the writes themselves and publish them system-wide
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            __threadfence_system();
        }
    }
}

// The common case, as straight-line code: the result goes out through TMA stores
// (beta == 0, C aligned), N is a multiple of 32 (a 32-column chunk is inside the
// matrix or outside it, never across its edge) and the bias, if any, can be read
// with 16-byte loads.  The output width class is a template parameter so that the
// staging layout is a compile-time constant.
constexpr int OUT32 = 0, OUT16 = 1;

template <int KIND, int BN, int STAGES, int CG, int EW, int ACTC, int OUTK>
__device__ __forceinline__ void epilogue_fast(const TcParams& p, const DestMaps* dests, const WaitCtx& wctx,
                                              uint32_t tmem_base, uint32_t acc_full_bar, uint32_t acc_empty_addr,
                                              uint32_t stage_addr, int warp, int lane, uint32_t cta_rank, int first_tile,
                                              int tile_step) {
    constexpr int EPI_BUFS = TileCfg<KIND, BN, STAGES, CG, EW>::EPI_BUFS;
    constexpr int NSPLIT = EW / 4;
    constexpr int CHUNKS = BN / (32 * NSPLIT);                         // 32-column chunks per warp in a whole tile
    // TMEM loads kept in flight while a chunk is processed: only where registers are plentiful (8 warps,
    // cheap activation); elsewhere the load and its wait are one step (PRE == 0)
    constexpr bool ASYNC_LD = (EW == 8) && (ACTC == ACTC_NONE || ACTC == ACTC_RELU);
    constexpr int PRE = ASYNC_LD ? (CHUNKS < EPI_PREFETCH ? CHUNKS : EPI_PREFETCH) : 0;
    constexpr int MODP = PRE > 0 ? PRE : 1;
    constexpr int EPI_COLS = (OUTK == OUT16 && BN / NSPLIT >= 64) ? 64 : 32; // columns per TMA store (host: TcParams::epi_cols)
    constexpr int SPG = EPI_COLS / 32;                                  // chunks per TMA store
    constexpr int ROWB = EPI_COLS * (OUTK == OUT16 ? 2 : 4);            // bytes per staging row: 128 or 64
    constexpr int C16 = (OUTK == OUT16) ? 4 : 8;                        // 16-byte pieces per 32 values
    const int lane_group = warp & 3;
    const int half = (warp - 2) >> 2;
    float alpha = p.alpha;
    if (p.scale_a_dev != nullptr) alpha /= __ldg(p.scale_a_dev);
    if (p.scale_b_dev != nullptr) alpha /= __ldg(p.scale_b_dev);
    const bool scaled = alpha != 1.0f;
    const bool has_bias = p.bias != nullptr;
    const bool bf16 = p.out_dtype == SM120_DTYPE_BFLOAT16;
    // this lane's staging row, and its swizzle term: 16-byte piece k of row r sits at piece k ^ (r & 7)
    // under the 128-byte swizzle and at k ^ ((r >> 1) & 3) under the 64-byte swizzle
    const uint32_t srow = stage_addr + static_cast<uint32_t>(lane) * ROWB;
    const uint32_t swz = static_cast<uint32_t>(ROWB == 128 ? (lane & 7) : ((lane >> 1) & 3)) << 4;
    uint32_t stores = 0;                                // TMA stores committed by this warp: picks the staging buffer
    int local = 0;
    for (int tile = first_tile; tile < p.num_work; tile += tile_step, ++local) {
        int bz, tm, n0, width;
        decode_work(tile, p, BN, bz, tm, n0, width);
        const uint32_t buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        const int row0 = (tm * CG + static_cast<int>(cta_rank)) * BM + lane_group * 32;   // first row of this warp
        const int cols_per_warp = width / NSPLIT;
        const int colbase = n0 + half * cols_per_warp;
        const int nvalid = max(0, min(cols_per_warp >> 5, (p.N - colbase) >> 5));          // chunks inside the matrix
        BiasRaw braw;
        if (has_bias && nvalid > 0) bias_prefetch32(p, colbase, braw);

        bool ok = mbar_wait(acc_full_bar + 8 * buf, acc_phase, wctx, 0x31000000u);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        if (p.trace != nullptr && warp == 2 && lane == 0 && local < TRACE_TILES)
            p.trace[static_cast<size_t>(blockIdx.x) * TRACE_WORDS + 8 + 4 * local + 2] = clock64();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + buf * BN + half * cols_per_warp;

        uint32_t acc[MODP][32];
        __syncwarp();
#pragma unroll
        for (int c = 0; c < PRE; ++c)
            if (c < nvalid) tmem_ld_32x32(t_row + c * 32, acc[c]);
        if (nvalid == 0) {
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_addr + 8 * buf);
        }
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            if (c < nvalid) {                               // warp-uniform
                const int col0 = colbase + c * 32;
                // loads were issued before step 0 and at every step s with s + PRE < nvalid
                if constexpr (PRE == 0) {
                    __syncwarp();
                    tmem_ld_32x32_sync(t_row + c * 32, acc[0]);
                    if (c == nvalid - 1) {                  // nothing more to load: hand the TMEM buffer back
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(acc_empty_addr + 8 * buf);
                    }
                } else if (c == 0 || (c - 1 + PRE < CHUNKS && c - 1 + PRE < nvalid)) {
#pragma unroll
                    for (int q = 0; q < PRE; ++q) tmem_ld_wait_regs(acc[q]);
                    if (c + PRE >= nvalid) {                // nothing more to load: hand the TMEM buffer back
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(acc_empty_addr + 8 * buf);
                    }
                }
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[c % MODP][j]);
                if (PRE > 0 && c + PRE < CHUNKS && c + PRE < nvalid) {
                    __syncwarp();
                    tmem_ld_32x32(t_row + (c + PRE) * 32, acc[c % MODP]);    // in flight while this chunk is processed
                }
                if (scaled) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] *= alpha;
                }
                if (has_bias) {
                    bias_add_raw32(p, col0, braw, v);
                    if (c + 1 < nvalid) bias_prefetch32(p, col0 + 32, braw);   // consumed one chunk later
                }
                act_apply32<ACTC>(v, p.activation);

                // Each warp stages and stores its own 32 rows: no barrier with the other warps.
                const int sub = (SPG == 2) ? (c & 1) : 0;              // position of this chunk in its store
                const bool last_of_store = (sub == SPG - 1) || (c == nvalid - 1);
                const uint32_t sbuf = (EPI_BUFS == 2) ? (stores & 1u) * EPI_STAGE_BYTES : 0u;
                if (sub == 0) {
                    // the staging buffer is about to be overwritten: the TMA store that last used it must have read it
                    if (lane == 0) bulk_wait_group_read<EPI_BUFS - 1>();
                    __syncwarp();
                }
                if constexpr (OUTK == OUT16) {
                    uint32_t packed[16];
                    pack16(v, bf16, packed);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        st_shared_v4(srow + sbuf + ((static_cast<uint32_t>(sub * C16 + k) << 4) ^ swz), packed[4 * k],
                                     packed[4 * k + 1], packed[4 * k + 2], packed[4 * k + 3]);
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        st_shared_v4(srow + sbuf + ((static_cast<uint32_t>(sub * C16 + k) << 4) ^ swz), __float_as_uint(v[4 * k]),
                                     __float_as_uint(v[4 * k + 1]), __float_as_uint(v[4 * k + 2]), __float_as_uint(v[4 * k + 3]));
                }
                if (last_of_store) {
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (row0 < p.M) {
                            for (int g = 0; g < p.num_dests; ++g)      // own C, then every peer's copy
                                tma_store_3d(&dests->m[g], stage_addr + sbuf, col0 - sub * 32, row0, bz);
                        }
                        bulk_commit_group();
                    }
                    ++stores;
                }
            }
        }
        if (p.trace != nullptr && warp == 2 && lane == 0 && local < TRACE_TILES)
            p.trace[static_cast<size_t>(blockIdx.x) * TRACE_WORDS + 8 + 4 * local + 3] = clock64();
    }
    if (lane == 0) {
        bulk_wait_group_read<0>();     // shared memory must outlive the stores that read it
        if (p.num_dests > 1) {
            // copies that went to other GPUs: wait for the writes themselves and publish them system-wide
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            __threadfence_system();
        }
    }
}

template <int KIND, int BN, int STAGES, int CG, int EW>
__global__ void __launch_bounds__(64 + 32 * EW, 1)
sm120_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                          const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_b_half,
                          const __grid_constant__ DestMaps dests,
                          const TcParams p) {
    using Cfg = TileCfg<KIND, BN, STAGES, CG, EW>;
    constexpr int EPB = Cfg::EPB, BK = Cfg::BK, UMMA_K = Cfg::UMMA_K, BN_CTA = Cfg::BN_CTA;
    constexpr uint32_t A_BYTES = Cfg::A_BYTES, STAGE_BYTES = Cfg::STAGE_BYTES, MN_BOX_BYTES = Cfg::MN_BOX_BYTES;
    constexpr uint32_t TMEM_COLS = Cfg::TMEM_COLS;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
    uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;                       // 1024-byte aligned
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + Cfg::EPI_BYTES);
    const uint32_t full_bar = smem_u32(bars);                       // [STAGES]
    const uint32_t empty_bar = smem_u32(bars + STAGES);             // [STAGES]
    const uint32_t acc_full_bar = smem_u32(bars + 2 * STAGES);      // [2]
    const uint32_t acc_empty_bar = smem_u32(bars + 2 * STAGES + 2); // [2]
    const uint32_t drain_bar = smem_u32(bars + 2 * STAGES + 4);     // [1]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
    volatile uint32_t* abort_flag = tmem_holder + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const long long probe_c0 = clock64();
    const unsigned long long probe_t0 = global_timer_ns();
    const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
    const bool leader = cta_rank == 0u;
    const int first_tile = (CG == 2) ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int tile_step = (CG == 2) ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    WaitCtx wctx{p.status, abort_flag, 0u, p.wait_limit_ns};
    if constexpr (CG == 2) wctx.peer_abort_addr = map_to_cta(smem_u32(const_cast<uint32_t*>(abort_flag)), cta_rank ^ 1u);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar + 8 * b, 1);
            mbar_init(acc_empty_bar + 8 * b, EW * CG);   // one arrival per epilogue warp of every CTA of the pair
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0u;
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        if (p.num_work > p.full_work) prefetch_tmap(&tmap_b_half);
        prefetch_tmap(&dests.m[0]);
    }
    if (warp == 1) {
        tmem_alloc<CG>(smem_u32(tmem_holder), TMEM_COLS);
        tmem_relinquish<CG>();
    }
    tcgen05_fence_before();
    __syncthreads();
    if constexpr (CG == 2) {       // the peer's barriers must exist before anything signals them
        cluster_arrive();
        cluster_wait();
    }
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    // Programmatic dependent launch: everything above touched only this CTA's shared memory and TMEM, so
    // it may run while the previous kernel of the stream drains; global memory is first touched after
    // the wait.  The next kernel of the stream may start its own set-up as soon as SMs free up.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (p.trace != nullptr && threadIdx.x == 0) {
        unsigned long long* t = p.trace + static_cast<size_t>(blockIdx.x) * TRACE_WORDS;
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        t[0] = probe_t0; t[1] = static_cast<unsigned long long>(probe_c0);
        t[2] = global_timer_ns(); t[3] = static_cast<unsigned long long>(clock64());
        t[7] = smid;
    }

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        // The whole warp runs the loop (so that its variables stay warp-uniform and
        // can live in uniform registers); one elected lane issues the copies.
        uint32_t stage = 0, phase = 0;
        long long issued = 0;
        bool ok = true;
        bool first = true;
        const uint32_t full_for_tma = (CG == 2) ? map_to_cta(full_bar, 0u) : full_bar;   // the pair leader's barriers
        for (int tile = first_tile; ok && tile < p.num_work; tile += tile_step) {
            int bz, tm, nt, width;
            decode_work(tile, p, BN, bz, tm, nt, width);
            const int za = p.a_batched ? bz : 0;
            const int zb = p.b_batched ? bz : 0;
            const int m0 = (tm * CG + static_cast<int>(cta_rank)) * BM;
            // this CTA's share of the tile's columns; a half-width tile loads only the rows of B that its
            // MMAs read (a box of half the height, or fewer boxes), which is what keeps the short last
            // wave from being bound by the bytes it pulls out of L2
            const int n0 = nt + static_cast<int>(cta_rank) * (width / CG);
            const bool half_item = tile >= p.full_work;
            const uint32_t stage_tx = Cfg::PARTS * (half_item ? (A_BYTES + p.b_bytes_half) : Cfg::PAIR_BYTES);
            for (int kb = 0; kb < p.k_blocks; ++kb) {
                if (first && kb == p.stall_kblock) { ok = false; break; }
                bool w = mbar_wait(empty_bar + 8 * stage, phase ^ 1u, wctx, 0x11000000u);
                w = __all_sync(0xFFFFFFFFu, w);
                if (!w) { ok = false; break; }
                if (elect_one_sync()) {
                    // transaction bytes of the whole pair are expected on the leader's barrier
                    if (leader) mbar_expect_tx(full_bar + 8 * stage, stage_tx * CG);
                    const uint32_t fb = full_for_tma + 8 * stage;
                    const uint32_t a_dst = smem_u32(smem) + stage * STAGE_BYTES;
                    const uint32_t b_dst = a_dst + A_BYTES;
                    const int k0 = bz * p.k_split + kb * BK;
                    if (!p.a_mn_major) {
                        tma_load_3d<CG>(a_dst, &tmap_a, fb, k0, m0, za);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / EPB; ++j)
                            tma_load_3d<CG>(a_dst + j * MN_BOX_BYTES, &tmap_a, fb, m0 + j * EPB, k0, za);
                    }
                    if constexpr (KIND == KIND_TF32) {
                        // the low pieces (the split operands are always K-major)
                        tma_load_3d<CG>(a_dst + Cfg::PAIR_BYTES, &tmap_a, fb, p.k_lo + k0, m0, za);
                        tma_load_3d<CG>(b_dst + Cfg::PAIR_BYTES, half_item ? &tmap_b_half : &tmap_b, fb, p.k_lo + k0, n0, zb);
                    }
                    if (!p.b_mn_major) {
                        tma_load_3d<CG>(b_dst, half_item ? &tmap_b_half : &tmap_b, fb, k0, n0, zb);
                    } else {
                        const int boxes = half_item ? p.b_boxes_half : BN_CTA / EPB;
#pragma unroll
                        for (int j = 0; j < BN_CTA / EPB; ++j)
                            if (j < boxes) tma_load_3d<CG>(b_dst + j * MN_BOX_BYTES, &tmap_b, fb, n0 + j * EPB, k0, zb);
                    }
                }
                __syncwarp();
                ++issued;
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            first = false;
        }
        // Before leaving, wait (bounded) until every copy issued has landed:
        // immediate on the normal path, where the MMA role consumed them all.
        // (Only the leader's barriers count transaction bytes.)
        if (leader) {
            const long long from = issued > STAGES ? issued - STAGES : 0;
            for (long long i = from; i < issued; ++i) {
                const uint32_t s = static_cast<uint32_t>(i % STAGES);
                const uint32_t par = static_cast<uint32_t>((i / STAGES) & 1);
                mbar_wait(full_bar + 8 * s, par, wctx, 0x13000000u, false);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) ------------------------------
        // Warp-uniform loop, one elected lane issues.  The 64-bit shared-memory
        // descriptors are kept as a constant high word and a low word that only
        // advances by the stage and K-step offsets.
        if (leader) {
            const uint32_t a_kstep = (p.a_mn_major ? static_cast<uint32_t>(UMMA_K) * 128u : 32u) >> 4;
            const uint32_t b_kstep = (p.b_mn_major ? static_cast<uint32_t>(UMMA_K) * 128u : 32u) >> 4;
            const uint32_t a_lo0 = ((smem_u32(smem) >> 4) & 0x3FFFu) | (((p.a_mn_major ? MN_BOX_BYTES : 16u) >> 4) << 16);
            const uint32_t b_lo0 = (((smem_u32(smem) + A_BYTES) >> 4) & 0x3FFFu) | (((p.b_mn_major ? MN_BOX_BYTES : 16u) >> 4) << 16);
            // high word: stride offset 1024 B (bits 32..45), version 1 (bits 46..47), 128-byte swizzle (bits 61..63)
            const uint64_t desc_hi = (static_cast<uint64_t>(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            bool issued_any = false;
            int local = 0;
            uint32_t acc_iter = 0;                          // accumulation runs issued so far: picks the TMEM buffer and the phase
            for (int tile = first_tile; ok && tile < p.num_work; tile += tile_step, ++local) {
                const uint32_t idesc = tile < p.full_work ? p.idesc : p.idesc_half;
                uint32_t buf = acc_iter & 1u;
                uint32_t d_tmem = tmem_base + buf * BN;
                int run_left = 0;                           // k-blocks left in the current accumulation run
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    bool w;
                    if (run_left == 0) {
                        // a new run (the only one of the tile, except on the fp32 path): its TMEM buffer must be free
                        if (kb != 0) {
                            if (elect_one_sync()) {         // the previous run is complete, in both CTAs of a pair
                                umma_commit<CG>(acc_full_bar + 8 * buf);
                                if constexpr (CG == 2) umma_commit<CG>(map_to_cta(acc_full_bar + 8 * buf, 1u));
                            }
                            __syncwarp();
                            ++acc_iter;
                        }
                        buf = acc_iter & 1u;
                        d_tmem = tmem_base + buf * BN;
                        w = mbar_wait(acc_empty_bar + 8 * buf, ((acc_iter >> 1) & 1u) ^ 1u, wctx, 0x21000000u);
                        w = __all_sync(0xFFFFFFFFu, w);
                        if (!w) { ok = false; break; }
                        tcgen05_fence_after();
                        run_left = p.kb_per_run;
                    }
                    const bool run_start = run_left == p.kb_per_run;
                    --run_left;
                    w = mbar_wait(full_bar + 8 * stage, phase, wctx, 0x22000000u);
                    w = __all_sync(0xFFFFFFFFu, w);
                    if (!w) { ok = false; break; }
                    tcgen05_fence_after();
                    if (p.trace != nullptr && kb == 0 && lane == 0 && local < TRACE_TILES)
                        p.trace[static_cast<size_t>(blockIdx.x) * TRACE_WORDS + 8 + 4 * local] = clock64();
                    const uint32_t soff = stage * (STAGE_BYTES >> 4);
                    if (elect_one_sync()) {
#pragma unroll
                        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                            const uint64_t a_desc = desc_hi | (a_lo0 + soff + kk * a_kstep);
                            const uint64_t b_desc = desc_hi | (b_lo0 + soff + kk * b_kstep);
                            umma_ss<KIND, CG>(d_tmem, a_desc, b_desc, idesc, (run_start && kk == 0) ? 0u : 1u);
                            if constexpr (KIND == KIND_TF32) {          // + A_hi . B_lo + A_lo . B_hi
                                constexpr uint32_t LO = Cfg::PAIR_BYTES >> 4;
                                umma_ss<KIND, CG>(d_tmem, a_desc, b_desc + LO, idesc, 1u);
                                umma_ss<KIND, CG>(d_tmem, a_desc + LO, b_desc, idesc, 1u);
                            }
                        }
                        // free the stage, in both CTAs of a pair, when these MMAs retire
                        umma_commit<CG>(empty_bar + 8 * stage);
                        if constexpr (CG == 2) umma_commit<CG>(map_to_cta(empty_bar + 8 * stage, 1u));
                    }
                    __syncwarp();
                    issued_any = true;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok && elect_one_sync()) {               // accumulator complete, in both CTAs of a pair
                    umma_commit<CG>(acc_full_bar + 8 * buf);
                    if constexpr (CG == 2) umma_commit<CG>(map_to_cta(acc_full_bar + 8 * buf, 1u));
                }
                __syncwarp();
                ++acc_iter;
                if (p.trace != nullptr && lane == 0 && local < TRACE_TILES)
                    p.trace[static_cast<size_t>(blockIdx.x) * TRACE_WORDS + 8 + 4 * local + 1] = clock64();
            }
            if (*abort_flag != 0u && issued_any) {
                if (elect_one_sync()) umma_commit<CG>(drain_bar);
                __syncwarp();
                mbar_wait(drain_bar, 0u, wctx, 0x23000000u, false);
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        uint32_t acc_empty_addr = acc_empty_bar;                       // the leader's barrier collects every arrival
        if constexpr (CG == 2) acc_empty_addr = map_to_cta(acc_empty_bar, 0u);
        const uint32_t stage_addr = smem_u32(epi_smem) + (warp - 2) * (Cfg::EPI_BUFS * EPI_STAGE_BYTES);   // this warp's staging buffers
#define SM120_EPI_ARGS p, &dests, wctx, tmem_base, acc_full_bar, acc_empty_addr, stage_addr, warp, lane, cta_rank, first_tile, tile_step
#define SM120_EPI_FAST(OUTK)                                                                                        \
    switch (p.activation) {                                                                                         \
        case SM120_ACTIVATION_NONE:     epilogue_fast<KIND, BN, STAGES, CG, EW, ACTC_NONE, OUTK>(SM120_EPI_ARGS); break;     \
        case SM120_ACTIVATION_RELU:     epilogue_fast<KIND, BN, STAGES, CG, EW, ACTC_RELU, OUTK>(SM120_EPI_ARGS); break;     \
        case SM120_ACTIVATION_GELU_ERF: epilogue_fast<KIND, BN, STAGES, CG, EW, ACTC_GELU_ERF, OUTK>(SM120_EPI_ARGS); break; \
        default:                        epilogue_fast<KIND, BN, STAGES, CG, EW, ACTC_DYNAMIC, OUTK>(SM120_EPI_ARGS); break;  \
    }
        if (p.fast_epi && KIND != KIND_TF32) {
            if (p.out_dtype == SM120_DTYPE_FLOAT32) { SM120_EPI_FAST(OUT32) } else { SM120_EPI_FAST(OUT16) }
        } else {
            epilogue_role<KIND, BN, STAGES, CG, EW, ACTC_DYNAMIC>(SM120_EPI_ARGS);
        }
#undef SM120_EPI_FAST
#undef SM120_EPI_ARGS
    }

    // ------------------------------ teardown ------------------------------
    tcgen05_fence_before();
    __syncthreads();
    if constexpr (CG == 2) {       // neither CTA may leave while its peer can still touch its shared memory or TMEM
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after();
        tmem_dealloc<CG>(tmem_base, TMEM_COLS);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        p.probe[0] = static_cast<unsigned long long>(clock64() - probe_c0);
        p.probe[1] = global_timer_ns() - probe_t0;
    }
    if (p.trace != nullptr && threadIdx.x == 0) {
        unsigned long long* t = p.trace + static_cast<size_t>(blockIdx.x) * TRACE_WORDS;
        int mine = 0;
        for (int tile = first_tile; tile < p.num_work; tile += tile_step) ++mine;
        t[4] = global_timer_ns(); t[5] = static_cast<unsigned long long>(clock64());
        t[6] = static_cast<unsigned long long>(mine);
    }
}


// Host helpers defined in gemm_tcgen05.cu, shared with the attention kernel: a cached 3-D tensor map with the
// 128-byte swizzle (extents, pitch and batch stride in elements), and the device's status words.
bool tc_encode_3d(CUtensorMap* map, const void* ptr, int dtype, int64_t inner, int64_t outer, int64_t nbatch, int64_t pitch,
                  int64_t bstride, uint32_t box_inner, uint32_t box_outer);
unsigned int* tc_status_address(int device);

// ---------------------------------------------------------------------------
// Host-side launch of one kernel variant.  Each variant is instantiated in its
// own translation unit (gemm_tcgen05_inst_*.cu) so that the variants compile in
// parallel; gemm_tcgen05.cu only declares them.
// ---------------------------------------------------------------------------
template <int KIND, int BN, int STAGES, int CG, int EW = 8>
cudaError_t launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb_half, const DestMaps& tc,
                           const TcParams& tp, int sm_count, int device, cudaStream_t stream, bool split_tail) {
    using Cfg = TileCfg<KIND, BN, STAGES, CG, EW>;
    static std::atomic<uint64_t> attr_done{0};     // one bit per device
    static std::atomic<int> max_clusters[64];      // CG == 2: co-resident clusters per device (0 = not asked yet)
    auto kern = sm120_gemm_tcgen05_kernel<KIND, BN, STAGES, CG, EW>;
    const uint64_t bit = 1ull << (device & 63);
    if ((attr_done.load(std::memory_order_acquire) & bit) == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::SMEM));
        if (e != cudaSuccess) return e;
        attr_done.fetch_or(bit, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // see griddepcontrol in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (CG == 2) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
        int clusters = max_clusters[device & 63].load(std::memory_order_acquire);
        if (clusters == 0) {
            cfg.gridDim = dim3(static_cast<unsigned>(sm_count & ~1), 1, 1);
            int n = 0;
            cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
            if (e != cudaSuccess) return e;
            if (n < 1) return cudaErrorInvalidConfiguration;
            clusters = n;
            max_clusters[device & 63].store(n, std::memory_order_release);
        }
        const int want = tp.num_tiles < clusters ? tp.num_tiles : clusters;
        cfg.gridDim = dim3(static_cast<unsigned>(2 * want), 1, 1);
        // A final wave that is less than half full is run as half-width tiles.
        TcParams t = tp;
        const int rest = tp.num_tiles % clusters;
        // (not with 16 epilogue warps: a warp's quarter of a half-width tile is narrower than its 64-column store)
        if (EW == 8 && tp.num_tiles > clusters && rest > 0 && 2 * rest <= clusters && split_tail) {
            t.full_work = tp.num_tiles - rest;
            t.num_work = t.full_work + 2 * rest;
        }
        return cudaLaunchKernelEx(&cfg, kern, ta, tb, tb_half, tc, t);
    } else {
        const int want = tp.num_tiles < sm_count ? tp.num_tiles : sm_count;
        cfg.gridDim = dim3(static_cast<unsigned>(want), 1, 1);
    }
    return cudaLaunchKernelEx(&cfg, kern, ta, tb, tb_half, tc, tp);
}


}  // namespace sm120
