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
// of 128.  384 threads in three warp groups:
//   warp 0     TMA producer: Q once, then K tiles (three-stage ring) and V tiles (two-stage ring)
//   warp 1     tcgen05.mma issuer and TMEM owner:
//                S_j  = Q K_j^T    (128 x 128, both operands K-major in shared memory) -> TMEM buffer j % 2
//                O_g += P_j V_j    (128 x D, g = j % 2; P_j is read FROM TENSOR MEMORY, where the softmax threads wrote it
//                                   over the last 64 columns of S_j;  V as stored: D contiguous) -> TMEM accumulator g
//              issue order  ... P_j V_j, S_{j+2}, P_{j+1} V_{j+1}, S_{j+3} ...: S_{j+2} overwrites the buffer that held
//              S_j and P_j, and the tensor pipe runs one thread's MMAs in the order they were issued, so it needs no wait.
//              P_j arrives in two halves of 64 keys with a barrier each, so the first four MMAs of P_j V_j start
//              while the second half is still being computed.
//   warps 2-3  idle (they complete warp group 0, which hands most of its registers to the other two groups)
//   warps 4-11 softmax, two GROUPS of four warps: group g owns the key tiles j with j % 2 = g, and with them S
//              buffer g and accumulator O_g.  Thread r of a group owns query row r (TMEM lane r) completely, so a tile
//              needs no exchange between threads: the 128 scores are read from TMEM into registers (232 per thread
//              after setmaxnreg), p = exp2(s - m) goes back into TMEM as packed bf16/fp16 pairs (the A operand of
//              P_j V_j), and the row sum is kept in a register.  The exponentials run in two straight runs of 64:
//              every asm volatile in between (a TMEM store, a fence) is a point the compiler cannot schedule across,
//              and each costs a drain of the MUFU pipeline.
//              m is the group's REFERENCE maximum of the row: it only moves when a tile's maximum exceeds it by more
//              than 8 (a factor 256 in p, harmless in 16 bits and in the fp32 sum); then the thread rescales its row
//              of O_g in TMEM, which is safe because "S_j is complete" implies that P_{j-2} V_{j-2}, the previous
//              product into O_g, is complete.  So O never passes through registers inside the loop.  The two groups
//              run half a period apart: one is in its exponentials (the MUFU unit) while the tensor pipe serves the
//              other.  At the end the groups exchange (m, l) per row through shared memory (a bounded wait on the
//              partner's sequence word), and each writes half of the columns of
//              (w_0 O_0 + w_1 O_1) / (w_0 l_0 + w_1 l_1).
// A group's period is its softmax time plus P_j V_j plus Q K_{j+2}^T (the next scores need the buffer that P_j lies
// in); TMEM (two score buffers + two accumulators = 512 columns at D = 128) has no room for a third score buffer
// that would take the products off that path.
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
constexpr int ATT_THREADS = 384;           // warp group 0: TMA, MMA and two idle warps; warp groups 1 and 2: softmax
constexpr int ATT_REGS_LOW = 40;            // registers per thread of warp group 0 after the hand-over
constexpr int ATT_REGS_HIGH = 232;          // ... of the softmax warp groups
constexpr int ATT_REGS_LAUNCH = 168;        // what the kernel must be compiled to (65536 / 384, rounded down to 8)
// setmaxnreg.inc waits, without a limit, for registers that warps of the SAME CTA have released: the eight softmax warps
// may only ask for what the four warps of group 0 give back
static_assert(8 * (ATT_REGS_HIGH - ATT_REGS_LAUNCH) <= 4 * (ATT_REGS_LAUNCH - ATT_REGS_LOW), "register hand-over does not balance");
constexpr float ATT_RESCALE_STEP = 8.0f;   // the reference maximum follows a tile's maximum only beyond this (log2 units)

// 2^x by the hardware unit (MUFU.EX2); -inf gives 0
__device__ __forceinline__ float att_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The two threads that share a query row (one per group) hand each other one float per step.  Thread (g, row)
// publishes value and step number; it then waits, bounded like every other wait of the kernel, until its partner has
// published the same step.  Values alternate between two slots, so a thread that is one step ahead never overwrites
// what its partner still has to read.
__device__ __forceinline__ bool pair_exchange(volatile float* vals, volatile int* seq, int g, int row, int step, float v,
                                              float& from_partner, const WaitCtx& w) {
    volatile float* slot = vals + (step & 1) * (2 * ATT_BM);
    const int mine = g * ATT_BM + row, other = (g ^ 1) * ATT_BM + row;
    slot[mine] = v;
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
    from_partner = slot[other];
    return true;
}

// The bounded mbarrier wait of the GEMM kernel, fully inlined: a warp whose register count was changed by
// setmaxnreg must not call a function that was compiled for the kernel's launch-time count.
__device__ __forceinline__ bool att_wait(uint32_t bar, uint32_t parity, const WaitCtx& w, uint32_t code, bool watch_abort = true) {
    if (mbar_try_wait(bar, parity)) return true;
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

// Two barriers that are both expected to be complete already: the two tests are in flight together, so the usual case
// costs one round trip to the barrier unit instead of two (the MMA-issuing thread's waits are on every tile's path)
__device__ __forceinline__ bool att_wait2(uint32_t bar_a, uint32_t parity_a, uint32_t bar_b, uint32_t parity_b, const WaitCtx& w,
                                          uint32_t code_a, uint32_t code_b) {
    const bool a = mbar_try_wait(bar_a, parity_a), b = mbar_try_wait(bar_b, parity_b);
    if (a && b) return true;
    if (!a && !att_wait(bar_a, parity_a, w, code_a)) return false;
    return b || att_wait(bar_b, parity_b, w, code_b);
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (M = 128 lanes x 16 K elements, two 16-bit elements per 32-bit cell)
// comes from tensor memory
__device__ __forceinline__ void umma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 TMEM lanes x 16 consecutive 32-bit columns -> 16 registers per thread; the registers are valid when it returns
__device__ __forceinline__ void tmem_ld_32x16_sync(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 (16) registers per thread -> 32 TMEM lanes x 32 (16) consecutive 32-bit columns (thread i of the warp owns
// lane i); complete after tmem_st_wait()
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
           "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
           "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
           "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
           "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

// Two fp32 values in one 64-bit register pair, and the packed fp32 arithmetic of sm_100 on them: one issue slot for
// two results
__device__ __forceinline__ uint64_t f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f32x2_split(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// the three-input maximum / minimum of sm_100: half the instructions and half the chain length of a row's search
__device__ __forceinline__ float att_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float att_min3(float a, float b, float c) {
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// p = exp2(s * scale_log2 - m) for KEYS of this thread's keys, packed as KEYS / 2 pairs of 16-bit values (the even key
// in the low half: the K-major A operand of P V); adds the exponentials to the pair of partial row sums l2.  EDGE: keys
// at or beyond key_limit count as 0 (only tiles that straddle the row's limit pay for the per-key tests).  The sum
// adds the unrounded exponentials: rounding each to 16 bits first costs two conversions per pair and changes the sum
// by a relative 2^-9 / sqrt(keys), far inside the output's own rounding.
template <int KEYS, bool EDGE>
__device__ __forceinline__ void att_exp_pack(const uint32_t (&s)[KEYS], uint32_t (&packed)[KEYS / 2], uint64_t scale2, uint64_t neg_m2,
                                             uint64_t& l2, int key0, int key_limit, bool bf16) {
#pragma unroll
    for (int i = 0; i < KEYS; i += 2) {
        const uint64_t x2 = fma2(f32x2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), scale2, neg_m2);
        float x0, x1;
        f32x2_split(x2, x0, x1);
        float p0 = att_exp2(x0), p1 = att_exp2(x1);
        if constexpr (EDGE) {
            if (key0 + i >= key_limit) p0 = 0.0f;
            if (key0 + i + 1 >= key_limit) p1 = 0.0f;
        }
        l2 = add2(l2, f32x2(p0, p1));
        if (bf16) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
        } else {
            const __half2 h = __floats2half2_rn(p0, p1);
            packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
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
    static constexpr uint32_t TILE_BYTES = Q_BYTES + ATT_K_STAGES * K_BYTES + ATT_V_STAGES * V_BYTES;
    // barriers + the row exchange: values [parity][group][row] and sequence words [group][row]
    static constexpr uint32_t BAR_BYTES = 256 + 2 * 2 * ATT_BM * 4 + 2 * ATT_BM * 4;
    static constexpr size_t SMEM_USED = TILE_BYTES + BAR_BYTES + 1024;
    // every CTA allocates all 512 TMEM columns, so two CTAs must never share an SM: request more than half of its shared memory
    static constexpr size_t SMEM = SMEM_USED > 118784 ? SMEM_USED : 118784;
    // S_0 at column 0, S_1 at 128 (P_j: the last 64 columns of S_j), O_0 at 256, O_1 at 256 + D
    static constexpr uint32_t TMEM_COLS = 512;
    static constexpr uint32_t TMEM_O = 2 * ATT_BN;
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
    const uint32_t v_smem = k_smem + ATT_K_STAGES * Cfg::K_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::TILE_BYTES);
    const uint32_t q_full = smem_u32(bars + 0);
    const uint32_t k_full = smem_u32(bars + 1);      // [3]
    const uint32_t k_empty = smem_u32(bars + 4);     // [3]
    const uint32_t v_full = smem_u32(bars + 7);      // [2]
    const uint32_t v_empty = smem_u32(bars + 9);     // [2]
    const uint32_t s_full = smem_u32(bars + 11);     // [2]  S_j is complete in TMEM (and with it every product issued before)
    const uint32_t p_lo = smem_u32(bars + 13);       // [2]  S_j has been read, keys 0-63 of P_j (and a rescaled O_g) are in TMEM
    const uint32_t p_hi = smem_u32(bars + 19);       // [2]  keys 64-127 of P_j are in TMEM
    const uint32_t o_done = smem_u32(bars + 15);     // [2]  the group's last product is complete
    const uint32_t drain_bar = smem_u32(bars + 17);
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 22);
    volatile uint32_t* abort_flag = tmem_holder + 1;
    volatile float* xchg = reinterpret_cast<volatile float*>(reinterpret_cast<uint8_t*>(bars) + 256);      // [2][2][ATT_BM]
    volatile int* xseq = reinterpret_cast<volatile int*>(reinterpret_cast<uint8_t*>(bars) + 256 + 2 * 2 * ATT_BM * 4);   // [2][ATT_BM]
    if (threadIdx.x < 2 * ATT_BM) xseq[threadIdx.x] = 0;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // Grid: (query tiles, batch), or with the causal mask (batch, query tiles) walked from the LAST query tile down:
    // a causal tile's work grows with its index, blocks are handed out in x-then-y order, so the long tiles of every
    // batch entry start first and the short ones fill the end of the launch
    const int q0 = (p.causal ? static_cast<int>(gridDim.y - 1 - blockIdx.y) : static_cast<int>(blockIdx.x)) * ATT_BM;
    const int bh = static_cast<int>(p.causal ? blockIdx.x : blockIdx.y);
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
            mbar_init(p_lo + 8 * b, 4);              // one arrival per warp of the group
            mbar_init(p_hi + 8 * b, 4);
            mbar_init(o_done + 8 * b, 1);
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0u;
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        // Q and the first two K tiles are requested here, before the TMEM allocation and the block-wide barrier below:
        // their trip from HBM is the longest part of a block's start, and nothing they need is still missing
        if (n_kv > 0) {
            mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
            for (int d = 0; d < DB; ++d) tma_load_3d<1>(q_smem + d * (ATT_BM * 128), &tmap_q, q_full, d * 64, q0, bh);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (j < n_kv) {
                    mbar_expect_tx(k_full + 8 * j, Cfg::K_BYTES);
#pragma unroll
                    for (int d = 0; d < DB; ++d)
                        tma_load_3d<1>(k_smem + j * Cfg::K_BYTES + d * (ATT_BN * 128), &tmap_k, k_full + 8 * j, d * 64, j * ATT_BN, bh);
                }
            }
        }
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(tmem_holder), Cfg::TMEM_COLS);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ATT_REGS_LOW));

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        bool ok = n_kv > 0;
        int issued_k = min(n_kv, 2), issued_v = 0;             // Q, K_0 and K_1 were requested during set-up
        auto load_k = [&](int j) -> bool {
            const uint32_t st = j % ATT_K_STAGES, ph = (j / ATT_K_STAGES) & 1;
            bool w = att_wait(k_empty + 8 * st, ph ^ 1u, wctx, 0x41000000u);
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
        // the scores run two tiles ahead of the P V products: K_0 and K_1 first (above), then V_j and K_{j+2}
        for (int j = 0; ok && j < n_kv; ++j) {
            const uint32_t st = j % ATT_V_STAGES, ph = (j / ATT_V_STAGES) & 1;
            bool w = att_wait(v_empty + 8 * st, ph ^ 1u, wctx, 0x42000000u);
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
        if (n_kv > 0) att_wait(q_full, 0u, wctx, 0x43000000u, false);
        for (int i = max(0, issued_k - ATT_K_STAGES); i < issued_k; ++i)
            att_wait(k_full + 8 * (i % ATT_K_STAGES), (i / ATT_K_STAGES) & 1, wctx, 0x43000000u, false);
        for (int i = max(0, issued_v - ATT_V_STAGES); i < issued_v; ++i)
            att_wait(v_full + 8 * (i % ATT_V_STAGES), (i / ATT_V_STAGES) & 1, wctx, 0x43000000u, false);
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        const uint32_t fmt = p.out_bf16 ? 1u : 0u;
        // M = 128; S: N = ATT_BN, both operands K-major; P V: N = D, A from TMEM, B (= V as stored) is N-major (bit 16)
        const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(ATT_BN >> 3) << 17) | (static_cast<uint32_t>(ATT_BM >> 4) << 24);
        const uint32_t idesc_pv = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | (static_cast<uint32_t>(D >> 3) << 17) | (static_cast<uint32_t>(ATT_BM >> 4) << 24);
        const uint64_t desc_hi = (static_cast<uint64_t>(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
        const uint32_t lbo_k = (16u >> 4) << 16;                   // K-major operands
        const uint32_t lbo_v = (8192u >> 4) << 16;                 // N-major V: 8 KB between its 64-column boxes
        bool ok = n_kv > 0;
        bool issued_any = false;
        if (ok) {
            bool w = att_wait(q_full, 0u, wctx, 0x51000000u);
            ok = __all_sync(0xFFFFFFFFu, w);
        }
        // S_j = Q K_j^T into S buffer j % 2.  The buffer is free: its last reader was P_{j-2} V_{j-2} (P_{j-2} lies in it),
        // issued by this thread before this product, and the softmax threads had read S_{j-2} before they wrote
        // P_{j-2}.
        // (One elected thread; the caller has waited for K_j.)
        auto qk_mmas = [&](int j) {
            const uint32_t st = j % ATT_K_STAGES, g = j & 1;
            const uint32_t s_tmem = tmem_base + g * ATT_BN;
#pragma unroll
            for (int t = 0; t < D / 16; ++t) {
                const uint32_t off = (t >> 2) * (128 * 128) + (t & 3) * 32;       // 64-element block, then 32 bytes per K step
                const uint64_t a_desc = desc_hi | ((((q_smem + off) >> 4) & 0x3FFFu) | lbo_k);
                const uint64_t b_desc = desc_hi | ((((k_smem + st * Cfg::K_BYTES + off) >> 4) & 0x3FFFu) | lbo_k);
                umma_ss<KIND_F16, 1>(s_tmem, a_desc, b_desc, idesc_s, t != 0 ? 1u : 0u);
            }
            umma_commit<1>(s_full + 8 * g);
            umma_commit<1>(k_empty + 8 * st);
        };
        // O_g += P_j[:, 16 t0 .. 16 t1) V_j[16 t0 .. 16 t1, :]   (one elected thread)
        auto pv_mmas = [&](int j, int t0, int t1) {
            const uint32_t g = j & 1, st = j % ATT_V_STAGES;
            const uint32_t p_tmem = tmem_base + g * ATT_BN + ATT_BN / 2;      // P_j: the upper 64 cells of S buffer g
            const uint32_t o_tmem = tmem_base + Cfg::TMEM_O + g * D;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                if (t < t0 || t >= t1) continue;
                const uint32_t b_off = (t >> 2) * (DB * 8192) + (t & 3) * 2048;   // 16 key rows of 128 bytes per K step
                const uint64_t b_desc = desc_hi | ((((v_smem + st * Cfg::V_BYTES + b_off) >> 4) & 0x3FFFu) | lbo_v);
                umma_ts_f16(o_tmem, p_tmem + t * 8, b_desc, idesc_pv, (t != 0 || j >= 2) ? 1u : 0u);   // 16 keys = 8 cells of P
            }
            if (t1 == 8) {
                umma_commit<1>(v_empty + 8 * st);
                if (j + 2 >= n_kv) umma_commit<1>(o_done + 8 * g);
            }
        };
        auto k_bar = [&](int j) { return k_full + 8 * (j % ATT_K_STAGES); };
        auto k_par = [&](int j) { return static_cast<uint32_t>((j / ATT_K_STAGES) & 1); };
        // The waits of this warp are on every tile's path (from "P_j is ready" to "S_{j+2} is issued"), and the warp
        // shares its scheduler with two busy softmax warps: barriers that are normally complete are tested in pairs,
        // and products that follow each other are issued from one election.
        for (int j0 = 0; ok && j0 < 2 && j0 < n_kv; ++j0) {
            bool w = att_wait(k_bar(j0), k_par(j0), wctx, 0x52000000u);
            ok = __all_sync(0xFFFFFFFFu, w);
            if (!ok) break;
            tcgen05_fence_after();
            if (elect_one_sync()) qk_mmas(j0);
            __syncwarp();
            issued_any = true;
        }
        for (int j = 0; ok && j < n_kv; ++j) {
            const uint32_t g = j & 1, bph = (j >> 1) & 1;
            const uint32_t vst = j % ATT_V_STAGES, vph = (j / ATT_V_STAGES) & 1;
            const bool more = j + 2 < n_kv;
            bool w = att_wait2(v_full + 8 * vst, vph, p_lo + 8 * g, bph, wctx, 0x54000000u, 0x55000000u);   // keys 0-63 of P_j are in TMEM
            ok = __all_sync(0xFFFFFFFFu, w);
            if (!ok) break;
            tcgen05_fence_after();
            if (elect_one_sync()) pv_mmas(j, 0, 4);
            __syncwarp();
            if (more) w = att_wait2(p_hi + 8 * g, bph, k_bar(j + 2), k_par(j + 2), wctx, 0x55000000u, 0x52000000u);
            else w = att_wait(p_hi + 8 * g, bph, wctx, 0x55000000u);
            ok = __all_sync(0xFFFFFFFFu, w);
            if (!ok) break;
            tcgen05_fence_after();
            if (elect_one_sync()) {
                pv_mmas(j, 4, 8);
                if (more) qk_mmas(j + 2);
            }
            __syncwarp();
        }
        if (*abort_flag != 0u && issued_any) {
            if (elect_one_sync()) umma_commit<1>(drain_bar);
            __syncwarp();
            att_wait(drain_bar, 0u, wctx, 0x57000000u, false);
        }
    } else if (warp >= 4) {
        // ------------------------------ softmax and output ------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(ATT_REGS_HIGH));
        const int lane_group = warp & 3;                       // TMEM lanes [32 * lane_group, +32)
        const int g = (warp - 4) >> 2;                         // group: key tiles j % 2 == g, S buffer g, accumulator O_g
        const int row = lane_group * 32 + lane;                // this thread's query row inside the tile
        const int q = q0 + row;
        const int key_limit = p.causal ? min(p.seq_k, q + p.seq_k - p.seq_q + 1) : p.seq_k;   // keys [0, key_limit) count
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
        const uint32_t t_s = t_lane + g * ATT_BN;              // S_j, and P_j in its last 64 cells
        const uint32_t t_o = t_lane + Cfg::TMEM_O + g * D;
        const bool bf16 = p.out_bf16 != 0;
        const float scale_log2 = p.scale_log2;
        float m_ref = -CUDART_INF_F, l_run = 0.0f;             // reference maximum (log2 units) and row sum relative to it
        bool ok = true;
        for (int j = g; j < n_kv; j += 2) {
            const int key0 = j * ATT_BN;
            ok = att_wait(s_full + 8 * g, (j >> 1) & 1, wctx, 0x61000000u);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            // the row's 128 scores -> registers; the tile's largest scaled score
            uint32_t s[ATT_BN];
            __syncwarp();
#pragma unroll
            for (int c = 0; c < ATT_BN / 32; ++c) tmem_ld_32x32(t_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
#pragma unroll
            for (int c = 0; c < ATT_BN / 32; ++c) tmem_ld_wait_regs(*reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
            const bool edge = key0 + ATT_BN > key_limit;        // some of the tile's keys do not count for this row
            // (the per-key tests exist only in the branch for tiles that straddle this row's key limit)
            float m_tile;
            if (!edge) {
                // four chains of three-input maxima; with a negative scale the largest scaled score belongs to the
                // smallest raw score
                float e0 = __uint_as_float(s[0]), e1 = __uint_as_float(s[1]), e2 = __uint_as_float(s[2]), e3 = __uint_as_float(s[3]);
                if (scale_log2 >= 0.0f) {
#pragma unroll
                    for (int i = 4; i + 8 <= ATT_BN; i += 8) {
                        e0 = att_max3(e0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
                        e1 = att_max3(e1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
                        e2 = att_max3(e2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
                        e3 = att_max3(e3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
                    }
                    e0 = att_max3(e0, __uint_as_float(s[ATT_BN - 4]), __uint_as_float(s[ATT_BN - 3]));
                    e1 = att_max3(e1, __uint_as_float(s[ATT_BN - 2]), __uint_as_float(s[ATT_BN - 1]));
                    m_tile = fmaxf(fmaxf(e0, e1), fmaxf(e2, e3)) * scale_log2;
                } else {
#pragma unroll
                    for (int i = 4; i + 8 <= ATT_BN; i += 8) {
                        e0 = att_min3(e0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
                        e1 = att_min3(e1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
                        e2 = att_min3(e2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
                        e3 = att_min3(e3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
                    }
                    e0 = att_min3(e0, __uint_as_float(s[ATT_BN - 4]), __uint_as_float(s[ATT_BN - 3]));
                    e1 = att_min3(e1, __uint_as_float(s[ATT_BN - 2]), __uint_as_float(s[ATT_BN - 1]));
                    m_tile = fminf(fminf(e0, e1), fminf(e2, e3)) * scale_log2;
                }
            } else {
                m_tile = -CUDART_INF_F;
#pragma unroll
                for (int i = 0; i < ATT_BN; ++i)
                    if (key0 + i < key_limit) m_tile = fmaxf(m_tile, __uint_as_float(s[i]) * scale_log2);
            }
            if (j < 2) {
                m_ref = m_tile;                                 // the group's first tile: O_g does not exist yet
            } else {
                // move the reference only when the tile exceeds it by more than ATT_RESCALE_STEP.  O_g may be rewritten
                // here: its last product (tile j - 2) was issued before S_j, which is complete.
                const bool moves = m_tile > m_ref + ATT_RESCALE_STEP;
                if (__any_sync(0xFFFFFFFFu, moves)) {
                    const float alpha = moves ? att_exp2(m_ref - m_tile) : 1.0f;     // 0 when the row had no key so far
#pragma unroll
                    for (int c = 0; c < D / 16; ++c) {
                        uint32_t oc[16];
                        tmem_ld_32x16_sync(t_o + c * 16, oc);
#pragma unroll
                        for (int i = 0; i < 16; ++i) oc[i] = __float_as_uint(__uint_as_float(oc[i]) * alpha);
                        tmem_st_32x32(t_o + c * 16, oc);
                    }
                    l_run *= alpha;
                    if (moves) m_ref = m_tile;
                }
            }
            const float m_use = m_ref == -CUDART_INF_F ? 0.0f : m_ref;      // a row without any key so far
            // p = exp2(s * scale_log2 - m), row sum, P (16-bit pairs) -> cells [64, 128) of the S buffer, whose scores are
            // in registers by now
            const uint64_t scale2 = f32x2(scale_log2, scale_log2), neg_m2 = f32x2(-m_use, -m_use);
            uint64_t l2 = f32x2(0.0f, 0.0f);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                // 64 keys at a time: one long run of independent exponentials, then one store; when half of P_j is
                // written its four MMAs may start
                uint32_t packed[32];
                const uint32_t(&sc)[64] = *reinterpret_cast<const uint32_t(*)[64]>(&s[c * 64]);
                if (edge) att_exp_pack<64, true>(sc, packed, scale2, neg_m2, l2, key0 + c * 64, key_limit, bf16);
                else att_exp_pack<64, false>(sc, packed, scale2, neg_m2, l2, key0 + c * 64, key_limit, bf16);
                tmem_st_32x32(t_s + ATT_BN / 2 + c * 32, packed);
                tmem_st_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive((c == 0 ? p_lo : p_hi) + 8 * g);
            }
            float l_a, l_b;
            f32x2_split(l2, l_a, l_b);
            l_run += l_a + l_b;
        }
        // both accumulators complete (a group without tiles has none: its weight below is 0 and its O is not read)
        const bool has0 = n_kv > 0, has1 = n_kv > 1;
        if (ok && has0) {
            ok = att_wait(o_done, 0u, wctx, 0x64000000u);
            ok = __all_sync(0xFFFFFFFFu, ok);
        }
        if (ok && has1) {
            ok = att_wait(o_done + 8, 0u, wctx, 0x64000000u);
            ok = __all_sync(0xFFFFFFFFu, ok);
        }
        // the row's true reference is the larger of the groups'; weights w_g = 2^(m_g - m), sum = w_0 l_0 + w_1 l_1
        float m_other = -CUDART_INF_F, lw_other = 0.0f;
        if (ok) ok = pair_exchange(xchg, xseq, g, row, 1, m_ref, m_other, wctx);
        const float m_all = fmaxf(m_ref, m_other);
        const float m_fin = m_all == -CUDART_INF_F ? 0.0f : m_all;
        const float w_mine = att_exp2(m_ref - m_fin), w_other = att_exp2(m_other - m_fin);      // 0 for a group without keys
        const float lw_mine = l_run * w_mine;
        if (ok) ok = pair_exchange(xchg, xseq, g, row, 2, lw_mine, lw_other, wctx);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (ok && n_kv > 0) {
            tcgen05_fence_after();
            const float l_row = g == 0 ? lw_mine + lw_other : lw_other + lw_mine;     // the same bits in both threads
            const float inv = l_row > 0.0f ? 1.0f / l_row : 0.0f;
            const float w0 = (g == 0 ? w_mine : w_other) * inv, w1 = (g == 0 ? w_other : w_mine) * inv;
            constexpr int HD = D / 2;                           // this thread writes columns [g * HD, +HD) of its row
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + (static_cast<size_t>(bh) * p.seq_q + q) * D + g * HD);
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t o0[32], o1[32];
                __syncwarp();
                tmem_ld_32x32_sync(t_lane + Cfg::TMEM_O + g * HD + c * 32, o0);
                if (has1) tmem_ld_32x32_sync(t_lane + Cfg::TMEM_O + D + g * HD + c * 32, o1);
                float r[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    r[i] = __uint_as_float(o0[i]) * w0;
                    if (has1) r[i] = fmaf(__uint_as_float(o1[i]), w1, r[i]);
                }
                if (q < p.seq_q) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint32_t w[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float a = r[v * 8 + 2 * k], b = r[v * 8 + 2 * k + 1];
                            if (bf16) {
                                const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                                w[k] = *reinterpret_cast<const uint32_t*>(&h);
                            } else {
                                const __half2 h = __floats2half2_rn(a, b);
                                w[k] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                        }
                        dst[c * 4 + v] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            tcgen05_fence_before();
        } else if (ok && q < p.seq_q) {
            // no key tile at all: the output row is 0
            constexpr int HD = D / 2;
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + (static_cast<size_t>(bh) * p.seq_q + q) * D + g * HD);
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) dst[c] = make_uint4(0u, 0u, 0u, 0u);
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
        // the register hand-over inside the kernel balances only if the kernel starts with ATT_REGS_LAUNCH registers
        cudaFuncAttributes fa{};
        cudaError_t e = cudaFuncGetAttributes(&fa, kern);
        if (e != cudaSuccess) return e;
        if (fa.numRegs != ATT_REGS_LAUNCH) return cudaErrorLaunchOutOfResources;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::SMEM));
        if (e != cudaSuccess) return e;
        attr_done.fetch_or(bit, std::memory_order_release);
    }
    const unsigned q_tiles = static_cast<unsigned>((p.seq_q + ATT_BM - 1) / ATT_BM), entries = static_cast<unsigned>(p.batch);
    const dim3 grid = p.causal ? dim3(entries, q_tiles, 1) : dim3(q_tiles, entries, 1);
    kern<<<grid, ATT_THREADS, Cfg::SMEM, stream>>>(tq, tk, tv, p);
    return cudaGetLastError();
}

bool attention_fused_supported(int dtype, long long batch, long long seq_q, long long seq_k, long long head_dim, const void* q,
                               const void* k, const void* v, const void* out) {
    if (dtype != SM120_DTYPE_FLOAT16 && dtype != SM120_DTYPE_BFLOAT16) return false;
    if (head_dim != 64 && head_dim != 128) return false;
    // batch entries and query tiles are grid dimensions, either of which may be the y dimension
    if (batch < 1 || batch > 65535 || seq_q < 1 || seq_k < 1 || seq_q > 65535ll * ATT_BM || seq_k >= (1ll << 31)) return false;
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
