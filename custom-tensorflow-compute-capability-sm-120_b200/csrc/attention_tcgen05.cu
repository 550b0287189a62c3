// Fused scaled-dot-product attention forward for B200 (sm_100a):
//     O = softmax(scale * Q K^T  [causal]) V        per (batch x head) entry
// in ONE kernel: both products run on the tcgen05 tensor cores with their
// accumulators in tensor memory, the softmax runs in registers between them, and
// the [seq, seq] score matrix never exists in HBM.  It is the fused form of the
// two batched GEMMs + softmax that the reference's attention layer issues
// (python/sm120_keras_layers.py:780-846, python/sm120_ops.py:385-402) and replaces
// its naive kernel (src/cuda_kernels/sm120_pure_kernels.cu:352-430, launcher
// src/cuda_kernels/sm120_c_interface.cu:232-268).
//
// One CTA owns 128 query rows of one batch entry and walks over the keys in tiles
// of 128.  64 + 128 SPLIT threads (SPLIT = threads per query row):
//   warp 0     TMA producer: Q once, then K tiles (three-stage ring) and V tiles (two-stage ring)
//   warp 1     tcgen05.mma issuer and TMEM owner:
//                S_j  = Q K_j^T   (128 x 128, both operands K-major in shared memory) -> TMEM, two buffers
//                PV_j = P_j V_j   (128 x D; P_j is read FROM TENSOR MEMORY, where the softmax threads wrote it
//                                  over the first 64 columns of S_j; V as stored: D contiguous) -> TMEM, two buffers
//              issue order  ... PV_j, S_{j+2}, PV_{j+1}, S_{j+3} ...: S_{j+2} overwrites the buffer that held S_j and
//              P_j, and the tensor pipe runs one thread's MMAs in the order they were issued, so it needs no wait.
//   the rest   softmax: query row r (TMEM lane r) belongs to SPLIT threads, one in each of the warps
//              w, w + 4, ... (all may read TMEM lanes 32 (w % 4) ..).  Each takes 128 / SPLIT of a tile's keys
//              and D / SPLIT of the output row.  Per key tile: the scores are read from TMEM in one go,
//              the partial row maxima are exchanged through shared memory (a bounded wait on the
//              partners' sequence words), p = exp2(s - m) goes as packed bf16/fp16 pairs back into TMEM as the A
//              operand of P_j V_j, and O = O * alpha + PV_{j-1} is accumulated in registers (the running output
//              row lives in registers, so nothing in TMEM is ever rescaled).  At the end O / l is written.
// While the softmax threads work on tile j the tensor pipe runs P_{j-1} V_{j-1} and Q K_{j+1}^T, and neither P nor
// the PV accumulator is shared between consecutive tiles, so the two sides only meet through the
// "P_j is written" and "S_j / PV_j is complete" barriers; the exponentials (one MUFU op per score) are what bounds
// the kernel.
//
// Every mbarrier wait is bounded like in the GEMM kernel (gemm_tcgen05_kernel.cuh): a wait
// that runs out records a status code, raises the CTA's abort flag, every role leaves its
// loop, outstanding copies and MMAs are drained with bounded waits, TMEM is freed and the
// kernel returns.

#include <cuda.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>
#include <atomic>

#include "gemm_tcgen05_kernel.cuh"

namespace sm120 {

constexpr int ATT_BM = 128;          // query rows per CTA
constexpr int ATT_BN = 128;          // keys per tile
constexpr int ATT_K_STAGES = 3;
constexpr int ATT_V_STAGES = 2;
#ifndef ATT_SPLIT_128
#define ATT_SPLIT_128 2                 // threads per query row at head dimension 128
#endif

// 2^x by the hardware unit (MUFU.EX2); -inf gives 0
__device__ __forceinline__ float att_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The SPLIT threads that share a query row hand each other one float per step (the partial row maximum of a key
// tile; at the end the partial row sum).  Thread `part` publishes value and step number; it then waits, bounded like
// every other wait of the kernel, until each partner has published the same step, and returns the maximum (MAX) or
// the sum in part order (so every partner gets the same bits).  Values alternate between two slots, so a thread
// that is one step ahead never overwrites what a partner still has to read.
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (M = 128 lanes x 16 K elements, two 16-bit elements per 32-bit cell)
// comes from tensor memory
__device__ __forceinline__ void umma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 registers per thread -> 32 TMEM lanes x 32 consecutive 32-bit columns (thread i of the warp owns lane i);
// returns when the store has completed
__device__ __forceinline__ void tmem_st_32x32_sync(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n\t"
        "tcgen05.wait::st.sync.aligned;"
        :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
           "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
           "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
           "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_32x32_sync(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n\t"
        "tcgen05.wait::st.sync.aligned;"
        :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
           "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

template <int SPLIT, bool MAX>
__device__ __forceinline__ bool group_exchange(volatile float* vals, volatile int* seq, int part, int row, int step, float v,
                                               float& combined, const WaitCtx& w) {
    volatile float* slot = vals + (step & 1) * (SPLIT * ATT_BM);
    slot[part * ATT_BM + row] = v;
    __threadfence_block();
    seq[part * ATT_BM + row] = step;
    float acc = MAX ? v : 0.0f;
#pragma unroll
    for (int o = 0; o < SPLIT; ++o) {
        if (o == part) {
            if (!MAX) acc += v;
            continue;
        }
        if (seq[o * ATT_BM + row] < step) {
            const unsigned long long t0 = global_timer_ns();
            uint32_t spins = 0;
            while (seq[o * ATT_BM + row] < step) {
                if ((++spins & 63u) == 0u) {
                    if (*w.abort_flag != 0u) return false;
                    if (global_timer_ns() - t0 > w.limit_ns) {
                        raise_abort(w, 0x65000000u);
                        return false;
                    }
                }
            }
        }
        __threadfence_block();
        const float x = slot[o * ATT_BM + row];
        acc = MAX ? fmaxf(acc, x) : acc + x;
    }
    combined = acc;
    return true;
}

// p = exp2(s * scale_log2 - m) for this thread's KEYS keys, packed as KEYS / 2 pairs of 16-bit values (the even key in the
// low half: the K-major A operand of P V); returns the row-sum contribution.  EDGE: keys at or beyond key_limit count
// as 0 (only tiles that straddle the row's limit pay for the per-key tests).  The sum adds the unrounded
// exponentials: rounding each to 16 bits first costs two conversions per pair and changes the sum by a relative
// 2^-9 / sqrt(keys), far inside the output's own rounding.
template <int KEYS, bool EDGE>
__device__ __forceinline__ float att_exp_pack(const uint32_t (&s)[KEYS], uint32_t (&packed)[KEYS / 2], float scale_log2, float m_use,
                                              int key0, int key_limit, bool bf16) {
    float l_a = 0.0f, l_b = 0.0f;
#pragma unroll
    for (int i = 0; i < KEYS; i += 2) {
        float p0 = att_exp2(fmaf(__uint_as_float(s[i]), scale_log2, -m_use));
        float p1 = att_exp2(fmaf(__uint_as_float(s[i + 1]), scale_log2, -m_use));
        if constexpr (EDGE) {
            if (key0 + i >= key_limit) p0 = 0.0f;
            if (key0 + i + 1 >= key_limit) p1 = 0.0f;
        }
        l_a += p0;
        l_b += p1;
        if (bf16) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
        } else {
            const __half2 h = __floats2half2_rn(p0, p1);
            packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    return l_a + l_b;
}

struct AttParams {
    int seq_q, seq_k, batch;         // batch = batch_size x heads
    int causal;                      // key k of query q is used when k <= q + seq_k - seq_q
    float scale_log2;                // scale * log2(e): the softmax works in base 2
    void* out;                       // [batch, seq_q, D], dense
    int out_bf16;
    unsigned long long wait_limit_ns;
    unsigned int* status;
};

// SPLIT = threads per query row: each takes ATT_BN / SPLIT keys of a tile and D / SPLIT columns of the output row
template <int D, int SPLIT>
struct AttCfg {
    static_assert(D == 64 || D == 128, "head dimension");
    static_assert((SPLIT == 2 || SPLIT == 4) && D / SPLIT >= 32, "threads per query row");
    static constexpr int THREADS = 64 + 128 * SPLIT;                  // TMA warp, MMA warp, 4 SPLIT softmax warps
    static constexpr uint32_t Q_BYTES = ATT_BM * D * 2;              // D/64 blocks of [128 rows x 128 B]
    static constexpr uint32_t K_BYTES = ATT_BN * D * 2;              // the same layout, ATT_BN rows
    static constexpr uint32_t V_BYTES = ATT_BN * D * 2;              // [ATT_BN/64 key blocks][D/64 boxes][64 keys x 128 B]
    static constexpr uint32_t TILE_BYTES = Q_BYTES + ATT_K_STAGES * K_BYTES + ATT_V_STAGES * V_BYTES;
    // barriers + the row exchange: values [parity][part][row] and sequence words [part][row]
    static constexpr uint32_t BAR_BYTES = 256 + 2 * SPLIT * ATT_BM * 4 + SPLIT * ATT_BM * 4;
    static constexpr size_t SMEM_USED = TILE_BYTES + BAR_BYTES + 1024;
    // every CTA allocates all 512 TMEM columns, so two CTAs must never share an SM: request more than half of its shared memory
    static constexpr size_t SMEM = SMEM_USED > 118784 ? SMEM_USED : 118784;
    // S_0 at column 0, S_1 at 128 (P_j: the first 64 columns of S_j), PV_0 at 256, PV_1 at 256 + D
    static constexpr uint32_t TMEM_COLS = 512;
    static constexpr uint32_t TMEM_PV = 2 * ATT_BN;
    static_assert(SMEM <= 232448, "shared memory budget exceeded");
};

template <int D, int SPLIT>
__global__ void __launch_bounds__(AttCfg<D, SPLIT>::THREADS, 1)
sm120_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q,
                               const __grid_constant__ CUtensorMap tmap_k,
                               const __grid_constant__ CUtensorMap tmap_v,
                               const AttParams p) {
    using Cfg = AttCfg<D, SPLIT>;
    constexpr int DB = D / 64;                       // 64-element (128-byte) blocks along the head dimension
    constexpr int KB = ATT_BN / 64;                  // 64-key blocks per key tile
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
    const uint32_t q_smem = smem_u32(smem);
    const uint32_t k_smem = q_smem + Cfg::Q_BYTES;
    const uint32_t v_smem = k_smem + ATT_K_STAGES * Cfg::K_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::TILE_BYTES);
    const uint32_t q_full = smem_u32(bars + 0);
    const uint32_t k_full = smem_u32(bars + 1);      // [3]
    const uint32_t k_empty = smem_u32(bars + 4);     // [3]
    const uint32_t v_full = smem_u32(bars + 7);      // [2]
    const uint32_t v_empty = smem_u32(bars + 9);     // [2]
    const uint32_t s_full = smem_u32(bars + 11);     // [2]  S_j is complete in TMEM
    const uint32_t p_full = smem_u32(bars + 13);     // [2]  S_j has been read and P_j is in TMEM
    const uint32_t pv_full = smem_u32(bars + 15);    // [2]  P_j V_j is complete in TMEM
    const uint32_t pv_empty = smem_u32(bars + 17);   // [2]  P_j V_j has been read
    const uint32_t drain_bar = smem_u32(bars + 19);
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 20);
    volatile uint32_t* abort_flag = tmem_holder + 1;
    volatile float* xchg = reinterpret_cast<volatile float*>(reinterpret_cast<uint8_t*>(bars) + 256);      // [2][SPLIT][ATT_BM]
    volatile int* xseq = reinterpret_cast<volatile int*>(reinterpret_cast<uint8_t*>(bars) + 256 + 2 * SPLIT * ATT_BM * 4);   // [SPLIT][ATT_BM]
    if (threadIdx.x < SPLIT * ATT_BM) xseq[threadIdx.x] = 0;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int q0 = static_cast<int>(blockIdx.x) * ATT_BM;
    const int bh = static_cast<int>(blockIdx.y);
    WaitCtx wctx{p.status, abort_flag, 0u, p.wait_limit_ns};

    // key tiles this CTA visits: all of them, or up to the diagonal of its last query row
    int n_kv = (p.seq_k + ATT_BN - 1) / ATT_BN;
    if (p.causal) {
        const int last_key = min(p.seq_k - 1, q0 + ATT_BM - 1 + p.seq_k - p.seq_q);
        n_kv = last_key < 0 ? 0 : min(n_kv, last_key / ATT_BN + 1);
    }

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int st = 0; st < ATT_K_STAGES; ++st) {
            mbar_init(k_full + 8 * st, 1);
            mbar_init(k_empty + 8 * st, 1);
        }
        for (int st = 0; st < ATT_V_STAGES; ++st) {
            mbar_init(v_full + 8 * st, 1);
            mbar_init(v_empty + 8 * st, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_full + 8 * b, 1);
            mbar_init(p_full + 8 * b, 4 * SPLIT);    // one arrival per softmax warp
            mbar_init(pv_full + 8 * b, 1);
            mbar_init(pv_empty + 8 * b, 4 * SPLIT);
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0u;
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(tmem_holder), Cfg::TMEM_COLS);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        bool ok = n_kv > 0;
        int issued_k = 0, issued_v = 0;
        if (ok && elect_one_sync()) {
            mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
            for (int d = 0; d < DB; ++d) tma_load_3d<1>(q_smem + d * (ATT_BM * 128), &tmap_q, q_full, d * 64, q0, bh);
        }
        __syncwarp();
        auto load_k = [&](int j) -> bool {
            const uint32_t st = j % ATT_K_STAGES, ph = (j / ATT_K_STAGES) & 1;
            bool w = mbar_wait(k_empty + 8 * st, ph ^ 1u, wctx, 0x41000000u);
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) return false;
            if (elect_one_sync()) {
                mbar_expect_tx(k_full + 8 * st, Cfg::K_BYTES);
#pragma unroll
                for (int d = 0; d < DB; ++d)
                    tma_load_3d<1>(k_smem + st * Cfg::K_BYTES + d * (ATT_BN * 128), &tmap_k, k_full + 8 * st, d * 64, j * ATT_BN, bh);
            }
            __syncwarp();
            ++issued_k;
            return true;
        };
        // the scores run two tiles ahead of the P V products: K_0 and K_1 first, then V_j and K_{j+2}
        if (ok) ok = load_k(0);
        if (ok && n_kv > 1) ok = load_k(1);
        for (int j = 0; ok && j < n_kv; ++j) {
            const uint32_t st = j % ATT_V_STAGES, ph = (j / ATT_V_STAGES) & 1;
            bool w = mbar_wait(v_empty + 8 * st, ph ^ 1u, wctx, 0x42000000u);
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) { ok = false; break; }
            if (elect_one_sync()) {
                mbar_expect_tx(v_full + 8 * st, Cfg::V_BYTES);
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                    for (int d = 0; d < DB; ++d)
                        tma_load_3d<1>(v_smem + st * Cfg::V_BYTES + (kb * DB + d) * 8192, &tmap_v, v_full + 8 * st, d * 64,
                                       j * ATT_BN + kb * 64, bh);
            }
            __syncwarp();
            ++issued_v;
            if (j + 2 < n_kv) ok = load_k(j + 2);
        }
        // before leaving: every copy issued must have landed (immediate unless the CTA is aborting)
        if (n_kv > 0) mbar_wait(q_full, 0u, wctx, 0x43000000u, false);
        for (int i = max(0, issued_k - ATT_K_STAGES); i < issued_k; ++i)
            mbar_wait(k_full + 8 * (i % ATT_K_STAGES), (i / ATT_K_STAGES) & 1, wctx, 0x43000000u, false);
        for (int i = max(0, issued_v - ATT_V_STAGES); i < issued_v; ++i)
            mbar_wait(v_full + 8 * (i % ATT_V_STAGES), (i / ATT_V_STAGES) & 1, wctx, 0x43000000u, false);
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        const uint32_t fmt = p.out_bf16 ? 1u : 0u;
        // M = 128; S: N = ATT_BN, both operands K-major; PV: N = D, A from TMEM, B (= V as stored) is N-major (bit 16)
        const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(ATT_BN >> 3) << 17) | (static_cast<uint32_t>(ATT_BM >> 4) << 24);
        const uint32_t idesc_pv = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | (static_cast<uint32_t>(D >> 3) << 17) | (static_cast<uint32_t>(ATT_BM >> 4) << 24);
        const uint64_t desc_hi = (static_cast<uint64_t>(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
        const uint32_t lbo_k = (16u >> 4) << 16;                   // K-major operands
        const uint32_t lbo_v = (8192u >> 4) << 16;                 // N-major V: 8 KB between its 64-column boxes
        bool ok = n_kv > 0;
        bool issued_any = false;
        if (ok) {
            bool w = mbar_wait(q_full, 0u, wctx, 0x51000000u);
            w = __all_sync(0xFFFFFFFFu, w);
            ok = w;
        }
        // S_j = Q K_j^T into S buffer j % 2.  The buffer is free: its last reader was P_{j-2} V_{j-2} (P_{j-2} lies
        // in it), issued by this thread before this product, and the softmax threads had read S_{j-2} before they
        // wrote P_{j-2}.
        auto issue_qk = [&](int j) -> bool {
            const uint32_t st = j % ATT_K_STAGES, ph = (j / ATT_K_STAGES) & 1;
            bool w = mbar_wait(k_full + 8 * st, ph, wctx, 0x52000000u);
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) return false;
            tcgen05_fence_after();
            if (elect_one_sync()) {
                const uint32_t d_tmem = tmem_base + (j & 1) * ATT_BN;
#pragma unroll
                for (int t = 0; t < D / 16; ++t) {
                    const uint32_t off = (t >> 2) * (128 * 128) + (t & 3) * 32;       // 64-element block, then 32 bytes per K step
                    const uint64_t a_desc = desc_hi | ((((q_smem + off) >> 4) & 0x3FFFu) | lbo_k);
                    const uint64_t b_desc = desc_hi | ((((k_smem + st * Cfg::K_BYTES + off) >> 4) & 0x3FFFu) | lbo_k);
                    umma_ss<KIND_F16, 1>(d_tmem, a_desc, b_desc, idesc_s, t != 0 ? 1u : 0u);
                }
                umma_commit<1>(s_full + 8 * (j & 1));
                umma_commit<1>(k_empty + 8 * st);
            }
            __syncwarp();
            issued_any = true;
            return true;
        };
        if (ok) ok = issue_qk(0);
        if (ok && n_kv > 1) ok = issue_qk(1);
        for (int j = 0; ok && j < n_kv; ++j) {
            const uint32_t b = j & 1, bph = (j >> 1) & 1;
            const uint32_t st = j % ATT_V_STAGES, ph = (j / ATT_V_STAGES) & 1;
            bool w = mbar_wait(v_full + 8 * st, ph, wctx, 0x54000000u);
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) { ok = false; break; }
            w = mbar_wait(p_full + 8 * b, bph, wctx, 0x55000000u);               // P_j is in TMEM
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) { ok = false; break; }
            w = mbar_wait(pv_empty + 8 * b, bph ^ 1u, wctx, 0x56000000u);        // P_{j-2} V_{j-2} has been read
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) { ok = false; break; }
            tcgen05_fence_after();
            if (elect_one_sync()) {
                const uint32_t d_tmem = tmem_base + Cfg::TMEM_PV + b * D;
                const uint32_t a_tmem = tmem_base + b * ATT_BN;
#pragma unroll
                for (int t = 0; t < ATT_BN / 16; ++t) {
                    const uint32_t b_off = (t >> 2) * (DB * 8192) + (t & 3) * 2048;   // 16 key rows of 128 bytes per K step
                    const uint64_t b_desc = desc_hi | ((((v_smem + st * Cfg::V_BYTES + b_off) >> 4) & 0x3FFFu) | lbo_v);
                    umma_ts_f16(d_tmem, a_tmem + t * 8, b_desc, idesc_pv, t != 0 ? 1u : 0u);   // 16 keys = 8 cells of P
                }
                umma_commit<1>(pv_full + 8 * b);
                umma_commit<1>(v_empty + 8 * st);
            }
            __syncwarp();
            if (j + 2 < n_kv) ok = issue_qk(j + 2);
        }
        if (*abort_flag != 0u && issued_any) {
            if (elect_one_sync()) umma_commit<1>(drain_bar);
            __syncwarp();
            mbar_wait(drain_bar, 0u, wctx, 0x57000000u, false);
        }
    } else {
        // ------------------------------ softmax and output ------------------------------
        constexpr int HD = D / SPLIT;                          // output columns per thread
        constexpr int KEYS = ATT_BN / SPLIT;                   // keys of a tile per thread
        const int lane_group = warp & 3;                       // TMEM lanes [32 * lane_group, +32)
        const int part = (warp - 2) >> 2;                      // which keys of a tile, which columns of the output row
        const int row = lane_group * 32 + lane;                // this thread's query row inside the tile
        const int q = q0 + row;
        const int key_limit = p.causal ? min(p.seq_k, q + p.seq_k - p.seq_q + 1) : p.seq_k;   // keys [0, key_limit) count
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
        float o[HD];
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] = 0.0f;
        float m_run = -CUDART_INF_F, l_run = 0.0f, alpha_prev = 1.0f;
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            const uint32_t b = j & 1, bph = (j >> 1) & 1;
            const int key0 = j * ATT_BN + part * KEYS;
            ok = mbar_wait(s_full + 8 * b, bph, wctx, 0x61000000u);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t t_s = t_lane + b * ATT_BN + part * KEYS;
            uint32_t s[KEYS];
            __syncwarp();
#pragma unroll
            for (int c = 0; c < KEYS / 32; ++c) tmem_ld_32x32(t_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
#pragma unroll
            for (int c = 0; c < KEYS / 32; ++c) tmem_ld_wait_regs(*reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
            const bool edge = key0 + KEYS > key_limit;          // some of this thread's keys do not count for this row
            // (the per-key tests exist only in the branch for tiles that straddle this row's key limit)
            float m_part = -CUDART_INF_F;
            if (!edge) {
                float ma = -CUDART_INF_F, mb = -CUDART_INF_F;       // two chains: the maxima do not depend on one another
#pragma unroll
                for (int i = 0; i < KEYS; i += 2) {
                    ma = fmaxf(ma, __uint_as_float(s[i]));
                    mb = fmaxf(mb, __uint_as_float(s[i + 1]));
                }
                m_part = fmaxf(ma, mb);
            } else {
#pragma unroll
                for (int i = 0; i < KEYS; ++i)
                    if (key0 + i < key_limit) m_part = fmaxf(m_part, __uint_as_float(s[i]));
            }
            // the row maximum of the tile: over this thread's keys and its partners'
            float m_tile = -CUDART_INF_F;
            ok = group_exchange<SPLIT, true>(xchg, xseq, part, row, j + 1, m_part, m_tile, wctx);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            const float m_new = fmaxf(m_run, m_tile * p.scale_log2);
            const float m_use = m_new == -CUDART_INF_F ? 0.0f : m_new;      // a row without any key so far
            const float alpha = att_exp2(m_run - m_use);                     // 0 for the first tile (m_run = -inf)
            // p = exp2(s * scale_log2 - m), partial row sum, P (16-bit pairs) -> TMEM cells [part * KEYS / 2, +KEYS / 2) of
            // the S buffer.  Those cells held scores of a partner's keys; the partner read them before it published
            // its maximum, and the exchange above has seen that.
            uint32_t packed[KEYS / 2];
            const float l_tile = edge ? att_exp_pack<KEYS, true>(s, packed, p.scale_log2, m_use, key0, key_limit, p.out_bf16 != 0)
                                      : att_exp_pack<KEYS, false>(s, packed, p.scale_log2, m_use, key0, key_limit, p.out_bf16 != 0);
            l_run = fmaf(l_run, alpha, l_tile);
            m_run = m_new;
            __syncwarp();
            tmem_st_32x32_sync(t_lane + b * ATT_BN + part * (KEYS / 2), packed);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 8 * b);
            // O_{j-1} = O_{j-2} * alpha_{j-1} + P_{j-1} V_{j-1}: that product finished long ago
            if (j > 0) {
                const uint32_t pb = (j - 1) & 1;
                ok = mbar_wait(pv_full + 8 * pb, ((j - 1) >> 1) & 1, wctx, 0x63000000u);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t pv[32];
                    __syncwarp();
                    tmem_ld_32x32_sync(t_lane + Cfg::TMEM_PV + pb * D + part * HD + c * 32, pv);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha_prev, __uint_as_float(pv[i]));
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(pv_empty + 8 * pb);
            }
            alpha_prev = alpha;
        }
        if (ok && n_kv > 0) {
            const uint32_t pb = (n_kv - 1) & 1;
            ok = mbar_wait(pv_full + 8 * pb, ((n_kv - 1) >> 1) & 1, wctx, 0x64000000u);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (ok) {
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t pv[32];
                    __syncwarp();
                    tmem_ld_32x32_sync(t_lane + Cfg::TMEM_PV + pb * D + part * HD + c * 32, pv);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha_prev, __uint_as_float(pv[i]));
                }
                tcgen05_fence_before();
            }
        }
        // the row sum is the sum of the partners' partial sums (all used the same maxima)
        float l_row = 0.0f;
        if (ok) ok = group_exchange<SPLIT, false>(xchg, xseq, part, row, n_kv + 1, l_run, l_row, wctx);
        if (ok && q < p.seq_q) {
            const float inv = l_row > 0.0f ? 1.0f / l_row : 0.0f;
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + (static_cast<size_t>(bh) * p.seq_q + q) * D + part * HD);
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float a = o[c * 8 + 2 * k] * inv, b = o[c * 8 + 2 * k + 1] * inv;
                    if (p.out_bf16) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                        w[k] = *reinterpret_cast<const uint32_t*>(&h);
                    } else {
                        const __half2 h = __floats2half2_rn(a, b);
                        w[k] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                }
                dst[c] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }

    // ------------------------------ teardown ------------------------------
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
    }
}

template <int D, int SPLIT>
static cudaError_t attention_launch_d(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttParams& p,
                                      int device, cudaStream_t stream) {
    using Cfg = AttCfg<D, SPLIT>;
    static std::atomic<uint64_t> attr_done{0};
    auto kern = sm120_attention_tcgen05_kernel<D, SPLIT>;
    const uint64_t bit = 1ull << (device & 63);
    if ((attr_done.load(std::memory_order_acquire) & bit) == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::SMEM));
        if (e != cudaSuccess) return e;
        attr_done.fetch_or(bit, std::memory_order_release);
    }
    const dim3 grid(static_cast<unsigned>((p.seq_q + ATT_BM - 1) / ATT_BM), static_cast<unsigned>(p.batch), 1);
    kern<<<grid, Cfg::THREADS, Cfg::SMEM, stream>>>(tq, tk, tv, p);
    return cudaGetLastError();
}

bool attention_fused_supported(int dtype, long long batch, long long seq_q, long long seq_k, long long head_dim, const void* q,
                               const void* k, const void* v, const void* out) {
    if (dtype != SM120_DTYPE_FLOAT16 && dtype != SM120_DTYPE_BFLOAT16) return false;
    if (head_dim != 64 && head_dim != 128) return false;
    if (batch < 1 || batch > 65535 || seq_q < 1 || seq_k < 1 || seq_q >= (1ll << 31) || seq_k >= (1ll << 31)) return false;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                           reinterpret_cast<uintptr_t>(out);
    return (bits & 15u) == 0;
}

// Q [batch, seq_q, D], K and V [batch, seq_k, D], out [batch, seq_q, D]: dense, 16-bit, D = 64 or 128.
cudaError_t attention_fused_launch(const void* q, const void* k, const void* v, void* out, long long batch, long long seq_q,
                                   long long seq_k, long long head_dim, float scale, int causal, int dtype, int device,
                                   uint64_t wait_limit_ns, cudaStream_t stream) {
    CUtensorMap tq, tk, tv;
    if (!tc_encode_3d(&tq, q, dtype, head_dim, seq_q, batch, head_dim, seq_q * head_dim, 64, ATT_BM)) return cudaErrorInvalidValue;
    if (!tc_encode_3d(&tk, k, dtype, head_dim, seq_k, batch, head_dim, seq_k * head_dim, 64, ATT_BN)) return cudaErrorInvalidValue;
    if (!tc_encode_3d(&tv, v, dtype, head_dim, seq_k, batch, head_dim, seq_k * head_dim, 64, 64)) return cudaErrorInvalidValue;
    AttParams p{};
    p.seq_q = static_cast<int>(seq_q); p.seq_k = static_cast<int>(seq_k); p.batch = static_cast<int>(batch);
    p.causal = causal;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = out;
    p.out_bf16 = dtype == SM120_DTYPE_BFLOAT16 ? 1 : 0;
    p.wait_limit_ns = wait_limit_ns;
    p.status = tc_status_address(device);
    if (p.status == nullptr) return cudaErrorInvalidSymbol;
    return head_dim == 128 ? attention_launch_d<128, ATT_SPLIT_128>(tq, tk, tv, p, device, stream)
                           : attention_launch_d<64, 2>(tq, tk, tv, p, device, stream);
}

}  // namespace sm120
