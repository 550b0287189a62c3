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
// of 128.  320 threads:
//   warp 0     TMA producer: Q once, then K and V tiles through two-stage rings
//   warp 1     tcgen05.mma issuer and TMEM owner:
//                S_j  = Q K_j^T        (128 x 128, K-major operands)       -> TMEM, double buffered
//                PV_j = P_j V_j        (128 x D; P from shared memory, V as stored: D contiguous) -> TMEM
//   warps 2-9  softmax: query row r (TMEM lane r) belongs to a PAIR of threads, one in warp w and one in
//              warp w + 4 (both may read TMEM lanes 32 (w % 4) ..).  Each takes 64 of a tile's 128 keys
//              and D / 2 of the output row.  Per key tile: the 64 scores are read from TMEM in one go,
//              the two partial row maxima are exchanged through shared memory (a bounded wait on the
//              partner's sequence word), p = exp2(s - m) goes as bf16/fp16 into shared memory as the A operand of
//              P_j V_j, and O = O * alpha + PV_{j-1} is accumulated in registers (the running output
//              row lives in registers, so nothing in TMEM is ever rescaled).  Two warps per scheduler
//              hide each other's TMEM, MUFU and shared-memory latencies.  At the end O / l is written.
// The score of tile j+1 is computed while P_j V_j runs and while the softmax warps work on
// tile j; the exponentials (one MUFU op per score) are what bounds the kernel.
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
constexpr int ATT_THREADS = 320;
constexpr int ATT_KV_STAGES = 2;

// 2^x by the hardware unit (MUFU.EX2); -inf gives 0
__device__ __forceinline__ float att_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The two threads that share a query row hand each other one float per step (the partial row maximum of a key
// tile; at the end the partial row sum).  Thread `mine` publishes value and step number; it then waits, bounded like
// every other wait of the kernel, until its partner has published the same step.  Values alternate between two
// slots, so a thread that is one step ahead never overwrites what its partner still has to read.
__device__ __forceinline__ bool pair_exchange(volatile float* vals, volatile int* seq, int mine, int other, int step, float v,
                                              float& from_partner, const WaitCtx& w) {
    vals[(step & 1) * (2 * ATT_BM) + mine] = v;
    __threadfence_block();
    seq[mine] = step;
    if (seq[other] < step) {
        const unsigned long long t0 = global_timer_ns();
        uint32_t spins = 0;
        while (seq[other] < step) {
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
    from_partner = vals[(step & 1) * (2 * ATT_BM) + other];
    return true;
}

// p = exp2(s * scale_log2 - m) for this thread's 64 keys, as 16-bit values into its 128-byte row of P (eight 16-byte
// pieces under the 128-byte swizzle); returns the row-sum contribution.  EDGE: keys at or beyond key_limit count as 0
// (only tiles that straddle the row's limit pay for the per-key tests).  The sum adds the unrounded exponentials:
// rounding each to 16 bits first costs two conversions per pair and changes the sum by a relative 2^-9 / sqrt(keys),
// far inside the output's own rounding.
template <bool EDGE>
__device__ __forceinline__ float att_exp_store(const uint32_t (&s0)[32], const uint32_t (&s1)[32], float scale_log2, float m_use,
                                               int key0, int key_limit, bool bf16, uint32_t p_row, uint32_t swz) {
    float l_a = 0.0f, l_b = 0.0f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            const float x0 = __uint_as_float(c == 0 ? s0[i] : s1[i]);
            const float x1 = __uint_as_float(c == 0 ? s0[i + 1] : s1[i + 1]);
            float p0 = att_exp2(fmaf(x0, scale_log2, -m_use));
            float p1 = att_exp2(fmaf(x1, scale_log2, -m_use));
            if constexpr (EDGE) {
                if (key0 + c * 32 + i >= key_limit) p0 = 0.0f;
                if (key0 + c * 32 + i + 1 >= key_limit) p1 = 0.0f;
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
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t piece = static_cast<uint32_t>(c * 4 + k);
            st_shared_v4(p_row + ((piece ^ swz) << 4), packed[4 * k], packed[4 * k + 1], packed[4 * k + 2], packed[4 * k + 3]);
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

template <int D>
struct AttCfg {
    static_assert(D == 64 || D == 128, "head dimension");
    static constexpr uint32_t Q_BYTES = ATT_BM * D * 2;              // D/64 blocks of [128 rows x 128 B]
    static constexpr uint32_t K_BYTES = ATT_BN * D * 2;              // the same layout, ATT_BN rows
    static constexpr uint32_t V_BYTES = ATT_BN * D * 2;              // [ATT_BN/64 key blocks][D/64 boxes][64 keys x 128 B]
    static constexpr uint32_t P_BYTES = ATT_BM * ATT_BN * 2;         // ATT_BN/64 blocks of [128 rows x 128 B]
    // barriers + the pair exchange: values [parity][half][row] and sequence words [half][row]
    static constexpr uint32_t BAR_BYTES = 256 + 2 * 2 * ATT_BM * 4 + 2 * ATT_BM * 4;
    static constexpr size_t SMEM_USED = Q_BYTES + ATT_KV_STAGES * (K_BYTES + V_BYTES) + P_BYTES + BAR_BYTES + 1024;
    // every CTA allocates all 512 TMEM columns, so two CTAs must never share an SM: request more than half of its shared memory
    static constexpr size_t SMEM = SMEM_USED > 118784 ? SMEM_USED : 118784;
    static constexpr uint32_t TMEM_COLS = 512;                        // S: 2 x 128 columns, PV: D columns at 256
    static_assert(SMEM <= 232448, "shared memory budget exceeded");
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
sm120_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q,
                               const __grid_constant__ CUtensorMap tmap_k,
                               const __grid_constant__ CUtensorMap tmap_v,
                               const AttParams p) {
    using Cfg = AttCfg<D>;
    constexpr int DB = D / 64;                       // 64-element (128-byte) blocks along the head dimension
    constexpr int KB = ATT_BN / 64;                  // 64-key blocks per key tile
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
    const uint32_t q_smem = smem_u32(smem);
    const uint32_t k_smem = q_smem + Cfg::Q_BYTES;
    const uint32_t v_smem = k_smem + ATT_KV_STAGES * Cfg::K_BYTES;
    const uint32_t p_smem = v_smem + ATT_KV_STAGES * Cfg::V_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::Q_BYTES + ATT_KV_STAGES * (Cfg::K_BYTES + Cfg::V_BYTES) + Cfg::P_BYTES);
    const uint32_t q_full = smem_u32(bars + 0);
    const uint32_t k_full = smem_u32(bars + 1);      // [2]
    const uint32_t k_empty = smem_u32(bars + 3);     // [2]
    const uint32_t v_full = smem_u32(bars + 5);      // [2]
    const uint32_t v_empty = smem_u32(bars + 7);     // [2]
    const uint32_t s_full = smem_u32(bars + 9);      // [2]
    const uint32_t s_empty = smem_u32(bars + 11);    // [2]
    const uint32_t p_full = smem_u32(bars + 13);
    const uint32_t p_empty = smem_u32(bars + 14);
    const uint32_t pv_full = smem_u32(bars + 15);
    const uint32_t pv_empty = smem_u32(bars + 16);
    const uint32_t drain_bar = smem_u32(bars + 17);
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 18);
    volatile uint32_t* abort_flag = tmem_holder + 1;
    volatile float* xchg = reinterpret_cast<volatile float*>(reinterpret_cast<uint8_t*>(bars) + 256);      // [2][2][ATT_BM]
    volatile int* xseq = reinterpret_cast<volatile int*>(reinterpret_cast<uint8_t*>(bars) + 256 + 2 * 2 * ATT_BM * 4);   // [2][ATT_BM]
    if (threadIdx.x < 2 * ATT_BM) xseq[threadIdx.x] = 0;

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
        for (int s = 0; s < 2; ++s) {
            mbar_init(k_full + 8 * s, 1);
            mbar_init(k_empty + 8 * s, 1);
            mbar_init(v_full + 8 * s, 1);
            mbar_init(v_empty + 8 * s, 1);
            mbar_init(s_full + 8 * s, 1);
            mbar_init(s_empty + 8 * s, 8);          // one arrival per softmax warp
        }
        mbar_init(p_full, 8);
        mbar_init(p_empty, 1);
        mbar_init(pv_full, 1);
        mbar_init(pv_empty, 8);
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
        for (int j = 0; ok && j < n_kv; ++j) {
            const uint32_t st = j & 1, ph = (j >> 1) & 1;
            const int key0 = j * ATT_BN;
            bool w = mbar_wait(k_empty + 8 * st, ph ^ 1u, wctx, 0x41000000u);
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) { ok = false; break; }
            if (elect_one_sync()) {
                mbar_expect_tx(k_full + 8 * st, Cfg::K_BYTES);
#pragma unroll
                for (int d = 0; d < DB; ++d)
                    tma_load_3d<1>(k_smem + st * Cfg::K_BYTES + d * (ATT_BN * 128), &tmap_k, k_full + 8 * st, d * 64, key0, bh);
            }
            __syncwarp();
            ++issued_k;
            w = mbar_wait(v_empty + 8 * st, ph ^ 1u, wctx, 0x42000000u);
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) { ok = false; break; }
            if (elect_one_sync()) {
                mbar_expect_tx(v_full + 8 * st, Cfg::V_BYTES);
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                    for (int d = 0; d < DB; ++d)
                        tma_load_3d<1>(v_smem + st * Cfg::V_BYTES + (kb * DB + d) * 8192, &tmap_v, v_full + 8 * st, d * 64,
                                       key0 + kb * 64, bh);
            }
            __syncwarp();
            ++issued_v;
        }
        // before leaving: every copy issued must have landed (immediate unless the CTA is aborting)
        if (n_kv > 0) mbar_wait(q_full, 0u, wctx, 0x43000000u, false);
        for (int i = max(0, issued_k - 2); i < issued_k; ++i) mbar_wait(k_full + 8 * (i & 1), (i >> 1) & 1, wctx, 0x43000000u, false);
        for (int i = max(0, issued_v - 2); i < issued_v; ++i) mbar_wait(v_full + 8 * (i & 1), (i >> 1) & 1, wctx, 0x43000000u, false);
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        const uint32_t fmt = p.out_bf16 ? 1u : 0u;
        // M = 128; S: N = ATT_BN, both operands K-major; PV: N = D, B (= V as stored) is N-major (bit 16)
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
        auto issue_qk = [&](int j) -> bool {
            const uint32_t st = j & 1, ph = (j >> 1) & 1;
            bool w = mbar_wait(k_full + 8 * st, ph, wctx, 0x52000000u);
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) return false;
            w = mbar_wait(s_empty + 8 * st, ph ^ 1u, wctx, 0x53000000u);       // S buffer j % 2 is free
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) return false;
            tcgen05_fence_after();
            if (elect_one_sync()) {
                const uint32_t d_tmem = tmem_base + st * ATT_BN;
#pragma unroll
                for (int t = 0; t < D / 16; ++t) {
                    const uint32_t off = (t >> 2) * (128 * 128) + (t & 3) * 32;       // 64-element block, then 32 bytes per K step
                    const uint64_t a_desc = desc_hi | ((((q_smem + off) >> 4) & 0x3FFFu) | lbo_k);
                    const uint64_t b_desc = desc_hi | ((((k_smem + st * Cfg::K_BYTES + off) >> 4) & 0x3FFFu) | lbo_k);
                    umma_ss<KIND_F16, 1>(d_tmem, a_desc, b_desc, idesc_s, t != 0 ? 1u : 0u);
                }
                umma_commit<1>(s_full + 8 * st);
                umma_commit<1>(k_empty + 8 * st);
            }
            __syncwarp();
            issued_any = true;
            return true;
        };
        if (ok) ok = issue_qk(0);
        for (int j = 0; ok && j < n_kv; ++j) {
            if (j + 1 < n_kv) {
                ok = issue_qk(j + 1);
                if (!ok) break;
            }
            const uint32_t st = j & 1, ph = (j >> 1) & 1;
            bool w = mbar_wait(v_full + 8 * st, ph, wctx, 0x54000000u);
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) { ok = false; break; }
            w = mbar_wait(p_full, j & 1, wctx, 0x55000000u);                    // P_j is in shared memory
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) { ok = false; break; }
            w = mbar_wait(pv_empty, (j & 1) ^ 1u, wctx, 0x56000000u);           // PV_{j-1} has been read
            w = __all_sync(0xFFFFFFFFu, w);
            if (!w) { ok = false; break; }
            tcgen05_fence_after();
            if (elect_one_sync()) {
                const uint32_t d_tmem = tmem_base + 2 * ATT_BN;
#pragma unroll
                for (int t = 0; t < ATT_BN / 16; ++t) {
                    const uint32_t a_off = (t >> 2) * (128 * 128) + (t & 3) * 32;
                    const uint32_t b_off = (t >> 2) * (DB * 8192) + (t & 3) * 2048;   // 16 key rows of 128 bytes per K step
                    const uint64_t a_desc = desc_hi | ((((p_smem + a_off) >> 4) & 0x3FFFu) | lbo_k);
                    const uint64_t b_desc = desc_hi | ((((v_smem + st * Cfg::V_BYTES + b_off) >> 4) & 0x3FFFu) | lbo_v);
                    umma_ss<KIND_F16, 1>(d_tmem, a_desc, b_desc, idesc_pv, t != 0 ? 1u : 0u);
                }
                umma_commit<1>(pv_full);
                umma_commit<1>(v_empty + 8 * st);
                umma_commit<1>(p_empty);
            }
            __syncwarp();
        }
        if (*abort_flag != 0u && issued_any) {
            if (elect_one_sync()) umma_commit<1>(drain_bar);
            __syncwarp();
            mbar_wait(drain_bar, 0u, wctx, 0x57000000u, false);
        }
    } else {
        // ------------------------------ softmax and output ------------------------------
        constexpr int HD = D / 2;                              // output columns per thread
        const int lane_group = warp & 3;                       // TMEM lanes [32 * lane_group, +32)
        const int half = (warp - 2) >> 2;                      // which 64 keys of a tile, which half of the output row
        const int row = lane_group * 32 + lane;                // this thread's query row inside the tile
        const int q = q0 + row;
        const int key_limit = p.causal ? min(p.seq_k, q + p.seq_k - p.seq_q + 1) : p.seq_k;   // keys [0, key_limit) count
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
        // this thread's 64 keys are the 128-byte row `row` of 64-key block `half` of P
        const uint32_t p_row = p_smem + static_cast<uint32_t>(half) * (128 * 128) + static_cast<uint32_t>(row) * 128u;
        const uint32_t swz = static_cast<uint32_t>(row & 7);
        const int xmine = half * ATT_BM + row, xother = (half ^ 1) * ATT_BM + row;   // this thread's and its partner's exchange slots
        float o[HD];
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] = 0.0f;
        float m_run = -CUDART_INF_F, l_run = 0.0f, alpha_prev = 1.0f;
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            const uint32_t st = j & 1, ph = (j >> 1) & 1;
            const int key0 = j * ATT_BN + half * 64;
            ok = mbar_wait(s_full + 8 * st, ph, wctx, 0x61000000u);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t t_s = t_lane + st * ATT_BN + half * 64;
            uint32_t s0[32], s1[32];
            __syncwarp();
            tmem_ld_32x32(t_s, s0);
            tmem_ld_32x32(t_s + 32, s1);
            tmem_ld_wait_regs(s0);
            tmem_ld_wait_regs(s1);
            tcgen05_fence_before();                             // S_j is in registers: the buffer may take S_{j+2}
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty + 8 * st);
            const bool edge = key0 + 64 > key_limit;            // some of this thread's keys do not count for this row
            // (the per-key tests exist only in the branch for tiles that straddle this row's key limit)
            float m_part = -CUDART_INF_F;
            if (!edge) {
                float ma = -CUDART_INF_F, mb = -CUDART_INF_F;       // two chains: the maxima do not depend on one another
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    ma = fmaxf(ma, __uint_as_float(s0[i]));
                    mb = fmaxf(mb, __uint_as_float(s1[i]));
                }
                m_part = fmaxf(ma, mb);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (key0 + i < key_limit) m_part = fmaxf(m_part, __uint_as_float(s0[i]));
                    if (key0 + 32 + i < key_limit) m_part = fmaxf(m_part, __uint_as_float(s1[i]));
                }
            }
            // the row maximum of the tile: this thread's 64 keys and its partner's
            float m_other = -CUDART_INF_F;
            ok = pair_exchange(xchg, xseq, xmine, xother, j + 1, m_part, m_other, wctx);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            const float m_tile = fmaxf(m_part, m_other);
            const float m_new = fmaxf(m_run, m_tile * p.scale_log2);
            const float m_use = m_new == -CUDART_INF_F ? 0.0f : m_new;      // a row without any key so far
            const float alpha = att_exp2(m_run - m_use);                     // 0 for the first tile (m_run = -inf)
            // the P buffer is free once P_{j-1} V_{j-1} has completed
            ok = mbar_wait(p_empty, (j & 1) ^ 1u, wctx, 0x62000000u);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            // p = exp2(s * scale_log2 - m), partial row sum, P -> shared memory (16-bit, 128-byte swizzle)
            const float l_tile = edge ? att_exp_store<true>(s0, s1, p.scale_log2, m_use, key0, key_limit, p.out_bf16 != 0, p_row, swz)
                                      : att_exp_store<false>(s0, s1, p.scale_log2, m_use, key0, key_limit, p.out_bf16 != 0, p_row, swz);
            l_run = fmaf(l_run, alpha, l_tile);
            m_run = m_new;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            // O_{j-1} = O_{j-2} * alpha_{j-1} + P_{j-1} V_{j-1}: that product finished long ago
            if (j > 0) {
                ok = mbar_wait(pv_full, (j - 1) & 1, wctx, 0x63000000u);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t pv[32];
                    __syncwarp();
                    tmem_ld_32x32_sync(t_lane + 2 * ATT_BN + half * HD + c * 32, pv);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha_prev, __uint_as_float(pv[i]));
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(pv_empty);
            }
            alpha_prev = alpha;
        }
        if (ok && n_kv > 0) {
            ok = mbar_wait(pv_full, (n_kv - 1) & 1, wctx, 0x64000000u);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (ok) {
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t pv[32];
                    __syncwarp();
                    tmem_ld_32x32_sync(t_lane + 2 * ATT_BN + half * HD + c * 32, pv);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha_prev, __uint_as_float(pv[i]));
                }
                tcgen05_fence_before();
            }
        }
        // the row sum is the sum of the pair's partial sums (both used the same maxima)
        float l_other = 0.0f;
        if (ok) ok = pair_exchange(xchg, xseq, xmine, xother, n_kv + 1, l_run, l_other, wctx);
        const float l_row = l_run + l_other;
        if (ok && q < p.seq_q) {
            const float inv = l_row > 0.0f ? 1.0f / l_row : 0.0f;
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + (static_cast<size_t>(bh) * p.seq_q + q) * D + half * HD);
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

template <int D>
static cudaError_t attention_launch_d(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttParams& p,
                                      int device, cudaStream_t stream) {
    using Cfg = AttCfg<D>;
    static std::atomic<uint64_t> attr_done{0};
    auto kern = sm120_attention_tcgen05_kernel<D>;
    const uint64_t bit = 1ull << (device & 63);
    if ((attr_done.load(std::memory_order_acquire) & bit) == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::SMEM));
        if (e != cudaSuccess) return e;
        attr_done.fetch_or(bit, std::memory_order_release);
    }
    const dim3 grid(static_cast<unsigned>((p.seq_q + ATT_BM - 1) / ATT_BM), static_cast<unsigned>(p.batch), 1);
    kern<<<grid, ATT_THREADS, Cfg::SMEM, stream>>>(tq, tk, tv, p);
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
    return head_dim == 128 ? attention_launch_d<128>(tq, tk, tv, p, device, stream) : attention_launch_d<64>(tq, tk, tv, p, device, stream);
}

}  // namespace sm120
