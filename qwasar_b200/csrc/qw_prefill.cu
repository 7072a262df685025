// Causal prefill attention over the bf16 KV cache: tcgen05 tensor cores, accumulators in
// tensor memory, operands staged by TMA (sm_100a).
//
// One CTA per (128-row query tile, query head).  K and V are read from the cache (the rows
// of this chunk were appended just before), 128 keys per step:
//
//   warp 9   TMA: K tiles   (two stages of 128 keys x 256 dims; 8 SWIZZLE_128B boxes of one page half each)
//   warp 10  TMA: V pages   (two stages of 64 keys x 256 dims: the two halves of a step)
//   warp 8   one thread issues tcgen05.mma:  S  = Q K_j^T   (M128 N128 K16 x 16: 8 with Q from TMEM, 8 from shared memory)
//   warp 11  one thread issues tcgen05.mma:  O += P_j V_j   (TS, M128 N256 K16 x 8,  P in TMEM)
//   warps 0-7  softmax: two threads per query row (= TMEM lane), 64 keys of every step each.  A
//            thread reads its scores from TMEM into registers and hands S back at once (so
//            Q K_{j+1}^T runs under this step's exponentials), online max / sum in the exp2
//            domain (the two halves swap their maxima through shared memory), writes P (bf16)
//            into tensor memory, rescales its half
//            of O in TMEM only when the row's max grew by more than 2^8, and at the end
//            normalises, applies the sigmoid output gate and stores its 128 dims of the row.
//            The exponentials are bounded by the special-function unit (16 per clock per SM,
//            half of a step's tensor time), so the step's critical chain -- read S, max,
//            exponentials, write P -- is split over two warps per scheduler.
//
// TMEM columns (512): O [0,256) fp32 | Q dims 0-127 [256,320) bf16 pairs | P [320,384) bf16 pairs |
// S [384,512) fp32.  Half of the query tile lives in tensor memory (as a shared-memory A operand it
// is re-read for every key tile); its other half, dims 128-255, stays in shared memory as a
// K-major swizzled operand, which frees the 64 columns the softmax weights P need: they go from
// registers straight into tensor memory (tcgen05.st) and are the A operand of P V from there, so no
// generic-proxy store to shared memory -- and none of the 500-clock proxy fence such stores need
// before the tensor core may read them -- sits on the step's critical chain.  Steps are 128
// keys wide because one thread issues every tcgen05.mma at roughly one per 65 clocks: a 64-key
// Q K^T step (32 clocks of tensor work) would be issue-bound.
// Every wait on an mbarrier is bounded (qw_common.cuh): a stuck pipeline ends the kernel with
// a status code instead of hanging the GPU, and TMEM is always released.
//
// FLOPs per (row, key): 4 * 256 (QK^T and PV), the count of tools/bench/fabench.c:37-38.
#include "qw_kernels.h"

namespace qw {

namespace {

constexpr int BM = 128, BN = 128;                     // query rows per CTA, keys per step
constexpr int K_BYTES = BN * 512;                     // 128 keys x 256 dims bf16
constexpr int KBOX = BN * 128;                        // one 64-dim box of a K tile (128 rows)
constexpr int V_BYTES = 64 * 512;                     // a V stage is one 64-key page
constexpr int VBOX = 64 * 128;
constexpr int P_BYTES = BM * BN * 2;                  // bf16 weights of one step, as an A operand
constexpr int PBOX = BM * 128;                        // 64 keys of every row
constexpr int OFF_K = 0, OFF_V = 2 * K_BYTES, OFF_P = OFF_V + 2 * V_BYTES, OFF_BAR = OFF_P + P_BYTES;
// Tiles that borrow the idle operand regions, all as SWIZZLE_128B boxes of 128 rows x 128 bytes
// (16 KB) moved by TMA.  In such a box a thread that owns one row touches 16-byte chunk c at
// c ^ (row & 7): eight neighbouring rows hit eight different bank groups, so the row-per-thread
// accesses below are conflict-free, and the transposition between "thread = row" and coalesced
// global rows is left to the copy engine.
//   Q tile (bf16, 4 boxes) in the V stages while the first K tile is already on its way;
//   gate tile (4 boxes bf16 / 8 boxes f32) in the K stages, loaded under the last step;
//   output tile written over the gate tile in place (same dtype), stored box by box.
constexpr int IO_BOX = BM * 128;
constexpr int OFF_STAGE_Q = OFF_V, OFF_STAGE_IO = OFF_K;
static_assert(4 * IO_BOX <= 2 * V_BYTES && 8 * IO_BOX <= 2 * K_BYTES, "staging overruns the operand regions");
constexpr int COL_O = 0, COL_Q = 256, COL_P = 320, COL_S = 384;    // TMEM columns
constexpr int OFF_QHI = OFF_P;                        // query dims 128-255: two K-major boxes of 128 rows x 64 dims
constexpr int OFF_CS = OFF_K + K_BYTES;               // the rows' cos / sin while the kernel norms its own tiles: in K stage 1
constexpr int OFF_XCH = OFF_BAR + 256;                // row maxima / sums passed between the two softmax halves
constexpr int OFF_WQ = OFF_XCH + 2 * 2 * BM * 4;      // the query norm weights (bf16 [256]) when the kernel norms its own tiles
constexpr int SMEM_BYTES = OFF_WQ + 512;              // the dynamic window is declared 1024-byte aligned
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB a CTA may use");
constexpr int THREADS = 12 * 32;                      // 8 softmax warps, Q K^T issue, K loads, V loads, P V issue
constexpr int W_MMA = 8, W_K = 9, W_V = 10, W_PV = 11;
#ifndef QW_QK_AFTER_PV
#define QW_QK_AFTER_PV 1
#endif
constexpr bool QK_AFTER_PV = QW_QK_AFTER_PV;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_BIG = -1.0e30f;
constexpr float RESCALE_AT = 8.0f;                    // log2 units

enum Bar { Q_READY = 0, Q_FULL, G_FULL, K_FULL0, K_FULL1, K_FREE0, K_FREE1, V_FULL0, V_FULL1, V_FREE0, V_FREE1,
           S_READY, S_FREE, P_READY, PV_DONE, PV_ISSUED, V_TAIL, N_BARS };

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- tcgen05 wrappers ---------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem].  The descriptor arrives as its two 32-bit halves (only the low
// one, which holds the start address, changes between steps) and ACC is a compile-time flag, so
// that one issue costs a handful of instructions: a single thread feeds the whole tensor pipe.
template <bool ACC>
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_tmem, uint32_t bdesc_lo, uint32_t bdesc_hi, uint32_t idesc) {
    if (ACC)
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\tsetp.eq.u32 p, 0, 0;\n\tmov.b64 bd, {%2, %3};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p;\n\t}"
            ::"r"(d), "r"(a_tmem), "r"(bdesc_lo), "r"(bdesc_hi), "r"(idesc) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\tsetp.ne.u32 p, 0, 0;\n\tmov.b64 bd, {%2, %3};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p;\n\t}"
            ::"r"(d), "r"(a_tmem), "r"(bdesc_lo), "r"(bdesc_hi), "r"(idesc) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
template <bool ACC>
__device__ __forceinline__ void mma_ss(uint32_t d, uint32_t adesc_lo, uint32_t adesc_hi, uint32_t bdesc_lo, uint32_t bdesc_hi,
                                       uint32_t idesc) {
    if (ACC)
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 ad, bd;\n\tsetp.eq.u32 p, 0, 0;\n\tmov.b64 ad, {%1, %2};\n\tmov.b64 bd, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], ad, bd, %5, p;\n\t}"
            ::"r"(d), "r"(adesc_lo), "r"(adesc_hi), "r"(bdesc_lo), "r"(bdesc_hi), "r"(idesc) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 ad, bd;\n\tsetp.ne.u32 p, 0, 0;\n\tmov.b64 ad, {%1, %2};\n\tmov.b64 bd, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], ad, bd, %5, p;\n\t}"
            ::"r"(d), "r"(adesc_lo), "r"(adesc_hi), "r"(bdesc_lo), "r"(bdesc_hi), "r"(idesc) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, SWIZZLE_128B (layout type 2), descriptor version 1, as halves:
// low = start address >> 4 (14 bits) | leading byte offset >> 4 at bit 16; high = stride byte
// offset >> 4 | version 1 at bit 14 | layout type 2 at bit 29.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
    return ((addr >> 4) & 0x3FFF) | (((lbo_bytes >> 4) & 0x3FFF) << 16);
}
__device__ __forceinline__ constexpr uint32_t desc_hi(uint32_t sbo_bytes) {
    return ((sbo_bytes >> 4) & 0x3FFF) | (1u << 14) | (2u << 29);
}
// kind::f16 instruction descriptor: fp32 accumulate, bf16 A and B.
__device__ __forceinline__ constexpr uint32_t instr_desc(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__global__ void __launch_bounds__(THREADS, 1) qw_attn_prefill_kernel(const __grid_constant__ PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {                      // swizzled boxes need 1024-byte alignment
        if (threadIdx.x == 0) report(p.status, QW_ST_BAD_SMEM);
        return;
    }
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + OFF_BAR);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + N_BARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heaviest tiles (latest rows) first; consecutive CTAs share the row tile and the kv head
    const int qt = p.n_q_tiles - 1 - (int)(blockIdx.x / p.q_heads);
    const int head = blockIdx.x % p.q_heads;
    const int kvh = head / p.gqa;
    const int q0 = qt * BM;
    const int n_keys = p.base_pos + p.rows;
    const int k_end = min(n_keys, p.base_pos + q0 + BM);          // keys any row of this tile may read
    const int n_t = (k_end + BN - 1) / BN;

    if (threadIdx.x == 0) {
        // the softmax side signals once per warp (lane 0, after the warp has converged)
        for (int i = 0; i < N_BARS; i++) mbar_init(&bars[i], (i == P_READY || i == S_FREE || i == Q_READY) ? 8 : 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == W_MMA) tmem_alloc(tmem_slot, 512);
    if (warp == W_K && p.fuse_q)                       // weights: 32 lanes x 8 bf16 (1.0 where there are none)
        reinterpret_cast<uint4 *>(smem + OFF_WQ)[lane] =
            p.q_norm_w ? __ldg(reinterpret_cast<const uint4 *>(p.q_norm_w) + lane) : make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_o = tmem + COL_O, t_q = tmem + COL_Q, t_p = tmem + COL_P, t_s = tmem + COL_S;

    // first row of the tensor map that holds page `pg` of this kv head (or a row past the map: zero fill)
    auto page_row = [&](const KvLayer &L, int pg) -> int32_t {
        if (pg * QW_PAGE_TOKENS >= n_keys) return p.oob_row;       // nothing of this page is visible: zeros, whatever memory holds
        if (L.table) {
            const int id = pg < L.pt_stride ? __ldg(L.table + (size_t)kvh * L.pt_stride + pg) : -1;
            return id >= 0 ? id * QW_PAGE_TOKENS : p.oob_row;
        }
        return pg * QW_PAGE_TOKENS < L.max_ctx ? kvh * L.max_ctx + pg * QW_PAGE_TOKENS : p.oob_row;
    };

    if (warp == W_K) {
        // ---------------- K tiles: two pages each, rows 0-63 and 64-127 of every 64-dim box ----------------
        if (lane == 0) {
            // Dependent launch: the cache rows of this chunk (and the rows' cos / sin) come from the
            // append kernel in front; everything a CTA does before this point -- barriers, tensor
            // memory, the raw query tile, which is an input of the node -- runs under that kernel's tail.
            pdl_wait();
            for (int j = 0; j < n_t; j++) {
                const int st = j & 1;
                const int32_t r0 = page_row(p.kc, 2 * j), r1 = page_row(p.kc, 2 * j + 1);
                if (j >= 2) mbar_wait(&bars[K_FREE0 + st], ((j >> 1) - 1) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
                if (j == 1 && p.fuse_q) mbar_wait(&bars[Q_READY], 0, abort_flag, p.status, QW_ST_MMA_TIMEOUT);   // stage 1 lent out, see OFF_CS
                mbar_expect_tx(&bars[K_FULL0 + st], K_BYTES);
                uint8_t *dst = smem + OFF_K + st * K_BYTES;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    tma_load_2d(dst + b * KBOX, &p.kmap, b * 64, r0, &bars[K_FULL0 + st]);
                    tma_load_2d(dst + b * KBOX + 8192, &p.kmap, b * 64, r1, &bars[K_FULL0 + st]);
                }
            }
            if (p.gate) {
                // the gate tile, into the K stages: both are idle once the last Q K^T has completed
                // (completions are in order), which is a whole step before the epilogue starts
                mbar_wait(&bars[K_FREE0 + ((n_t - 1) & 1)], ((n_t - 1) >> 1) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
                const int n_box = p.gate_dtype == DT_BF16 ? 4 : 8, w = p.gate_dtype == DT_BF16 ? 64 : 32;
                mbar_expect_tx(&bars[G_FULL], n_box * IO_BOX);
                for (int b = 0; b < n_box; b++)
                    tma_load_2d(smem + OFF_STAGE_IO + b * IO_BOX, &p.gmap, head * p.gate_stride + b * w, q0, &bars[G_FULL]);
            }
        }
    } else if (warp == W_V) {
        // ---------------- V pages ----------------
        if (lane == 0) {
            // the Q tile (raw q rows of the [q|gate] input when the kernel norms and rotates them
            // itself, then together with the rows' cos / sin, parked in the P region)
            mbar_expect_tx(&bars[Q_FULL], (p.fuse_q ? 6 : 4) * IO_BOX);
            if (!p.fuse_q) pdl_wait();                     // ready-made queries are written by the kernel in front
            // ready-made queries: dims 0-127 to the staging area (they move on to tensor memory),
            // dims 128-255 straight to where the tensor core reads them; raw rows: all four boxes to
            // the staging area, their cos / sin to K stage 1
#pragma unroll
            for (int b = 0; b < 4; b++)
                tma_load_2d(smem + ((p.fuse_q || b < 2) ? OFF_STAGE_Q + b * IO_BOX : OFF_QHI + (b - 2) * IO_BOX), &p.qmap,
                            head * (p.fuse_q ? 512 : 256) + b * 64, q0, &bars[Q_FULL]);
            if (p.fuse_q) {
                pdl_wait();                                // the raw rows above are inputs; the angles are not
                tma_load_2d(smem + OFF_CS, &p.csmap, 0, q0, &bars[Q_FULL]);
                tma_load_2d(smem + OFF_CS + IO_BOX, &p.csmap, 32, q0, &bars[Q_FULL]);
            }
            mbar_wait(&bars[Q_READY], 0, abort_flag, p.status, QW_ST_MMA_TIMEOUT);   // the Q tile borrowed this region
            for (int pg = 0; pg < 2 * n_t; pg++) {
                const int st = pg & 1;
                const int32_t r = page_row(p.vc, pg);
                if (pg >= 2) mbar_wait(&bars[V_FREE0 + st], ((pg >> 1) - 1) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
                mbar_expect_tx(&bars[V_FULL0 + st], V_BYTES);
#pragma unroll
                for (int b = 0; b < 4; b++)
                    tma_load_2d(smem + OFF_V + st * V_BYTES + b * VBOX, &p.vmap, b * 64, r, &bars[V_FULL0 + st]);
            }
        }
        __syncwarp();
        // The page that holds the last key: its rows past that key may hold anything (a recycled
        // page, a caller's own buffer), and although their softmax weights are exactly 0, 0 x NaN
        // would still poison the whole output tile.  The warp clears those rows in shared memory
        // once the page has landed, and the P V issuer waits for that before it uses the page.
        // (The page is one of the last two of this tile, so its stage is not filled again.)
        const int pg_r = n_keys >> 6;
        if ((n_keys & 63) && pg_r < 2 * n_t) {
            mbar_wait(&bars[V_FULL0 + (pg_r & 1)], (pg_r >> 1) & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
            uint8_t *stg = smem + OFF_V + (pg_r & 1) * V_BYTES;
#pragma unroll
            for (int b = 0; b < 4; b++)
                for (int off = (n_keys & 63) * 128 + lane * 16; off < 64 * 128; off += 32 * 16)
                    *reinterpret_cast<uint4 *>(stg + b * VBOX + off) = make_uint4(0, 0, 0, 0);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[V_TAIL]);
        }
    } else if (warp == W_MMA) {
        // ---------------- tensor-core issue, S = Q K^T ----------------
        // The two products are issued by two threads (this one and warp W_PV): a thread that has
        // just queued tensor work is slow to get through its next barrier, and with one issuer
        // those pauses (five per step) left the tensor pipe idle for almost half of the step.
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc(128, BN, 0);
            constexpr uint32_t hi = desc_hi(1024);
            const uint32_t k_a = smem_u32(smem + OFF_K);
            const uint32_t qh_lo = desc_lo(smem_u32(smem + OFF_QHI), 16);
            mbar_wait(&bars[Q_READY], 0, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
            for (int j = 0; j < n_t; j++) {
                const int st = j & 1;
                // S is handed back as soon as the softmax threads hold step j-1 in registers
                // The waits that are normally over long before come first: even a satisfied wait
                // costs a few hundred clocks here.
                mbar_wait_hot(&bars[K_FULL0 + st], (j >> 1) & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                if (j > 0) mbar_wait_hot(&bars[S_FREE], (j - 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
                // P V of step j-2 goes into the tensor queue first: queued side by side the two
                // products share the pipe, and the softmax threads wait for the end of P V before
                // they may write the next P -- which they then do under this product.
                if (QK_AFTER_PV && j > 1) mbar_wait_hot(&bars[PV_ISSUED], j & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
                tc_fence_after();
                const uint32_t k_lo = desc_lo(k_a + st * K_BYTES, 16);
                // A: 16 dims of Q = 8 TMEM columns for dims 0-127, 32 bytes inside the swizzle atom of a
                // shared-memory box for dims 128-255; B: 16 dims = 32 bytes (2 units) inside the swizzle
                // atom, 64 dims per box (KBOX / 16 units)
                mma_ts<false>(t_s, t_q, k_lo, hi, idesc_qk);
#pragma unroll
                for (int ks = 1; ks < 8; ks++)
                    mma_ts<true>(t_s, t_q + ks * 8, k_lo + (ks >> 2) * (KBOX >> 4) + (ks & 3) * 2, hi, idesc_qk);
#pragma unroll
                for (int ks = 8; ks < 16; ks++)
                    mma_ss<true>(t_s, qh_lo + ((ks - 8) >> 2) * (IO_BOX >> 4) + (ks & 3) * 2, hi,
                                 k_lo + (ks >> 2) * (KBOX >> 4) + (ks & 3) * 2, hi, idesc_qk);
                tc_commit(&bars[S_READY]);
                tc_commit(&bars[K_FREE0 + st]);
            }
        }
    } else if (warp == W_PV) {
        // ---------------- tensor-core issue, O += P V ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_pv = instr_desc(128, 256, 1);
            constexpr uint32_t hi = desc_hi(1024);
            const uint32_t v_a = smem_u32(smem + OFF_V);
            for (int j = 0; j < n_t; j++) {
                // the first V page (normally there already), then the weights; the second page
                // was requested only when the step before ended and lands under the first half
                mbar_wait_hot(&bars[V_FULL0], j & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                mbar_wait_hot(&bars[P_READY], j & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < 2; h++) {                  // the two 64-key pages of the step
                    if (h == 1) {
                        mbar_wait_hot(&bars[V_FULL1], j & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                        tc_fence_after();
                    }
                    if ((n_keys & 63) && 2 * j + h == (n_keys >> 6)) {      // the page with the last key: cleared past it first
                        mbar_wait(&bars[V_TAIL], 0, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                        tc_fence_after();
                    }
                    const uint32_t v_lo = desc_lo(v_a + h * V_BYTES, VBOX);
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) {
                        // A: 16 keys of P = 8 TMEM columns; B: 16 keys of V = 2048 bytes
                        const uint32_t a_p = t_p + (h * 4 + ks) * 8;
                        if (j > 0 || h > 0 || ks > 0) mma_ts<true>(t_o, a_p, v_lo + ks * 128, hi, idesc_pv);
                        else mma_ts<false>(t_o, a_p, v_lo + ks * 128, hi, idesc_pv);
                    }
                    tc_commit(&bars[V_FREE0 + h]);
                }
                tc_commit(&bars[PV_DONE]);
                if (QK_AFTER_PV) mbar_arrive(&bars[PV_ISSUED]);
            }
        }
    } else {
        // ---------------- softmax + epilogue ----------------
        // Two threads per query row (= TMEM lane): warps 0-3 take keys 0-63 of every step and
        // output dims 0-127, warps 4-7 keys 64-127 and dims 128-255 (a warp reaches the 32 lanes
        // of its index modulo 4).  The halves exchange their row maxima through shared memory, so
        // both follow the same running max and rescale decisions; each keeps the sum of its keys.
        const int wg = warp >> 2;
        const int row_l = (warp & 3) * 32 + lane;
        const int row_g = q0 + row_l;
        const bool valid = row_g < p.rows;
        const int limit = valid ? p.base_pos + row_g : 0x7fffffff;         // last key this row may read
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const float sc2 = p.scale * LOG2E;
        float *xch = reinterpret_cast<float *>(smem + OFF_XCH);             // [2][2][BM]
        float m = NEG_BIG, l = 0.0f;
        uint32_t v[32];
        const uint32_t sw = row_l & 7;
        {
            // The Q tile arrives by TMA.  Dims 0-127 (two boxes = 64 columns of bf16 pairs) are moved
            // into the row's TMEM lane by the first of the row's two threads; dims 128-255 stay in
            // shared memory (ready-made queries were delivered there, raw rows are normed and put
            // there by the row's second thread).  Rows past the end of the chunk read as zeros.
            const uint8_t *q_row = smem + OFF_STAGE_Q + row_l * 128;
            mbar_wait(&bars[Q_FULL], 0, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
            if (!p.fuse_q) {
#pragma unroll
                for (int c = 0; c < 2 * (1 - wg); c++) {
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const uint4 x = *reinterpret_cast<const uint4 *>(q_row + c * IO_BOX + ((e ^ sw) << 4));
                        v[e * 4] = x.x; v[e * 4 + 1] = x.y; v[e * 4 + 2] = x.z; v[e * 4 + 3] = x.w;
                    }
                    tmem_st32(t_q + lane_base + c * 32, v);
                }
            } else {
                // Per-head RMS norm and partial RoPE of the raw rows, operation for operation as the
                // pre-op does them (qwasar_cpu.c:68-82, 304-319) except for the order of the sum of
                // squares: each of the row's two threads sums its 128 dims, the halves are added.
                float ss = 0.0f;
#pragma unroll
                for (int c = 2 * wg; c < 2 * wg + 2; c++) {
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const uint4 x = *reinterpret_cast<const uint4 *>(q_row + c * IO_BOX + ((e ^ sw) << 4));
                        const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const float lo = __uint_as_float(xw[i] << 16), hi = __uint_as_float(xw[i] & 0xffff0000u);
                            ss = __fadd_rn(ss, __fmul_rn(lo, lo));
                            ss = __fadd_rn(ss, __fmul_rn(hi, hi));
                        }
                    }
                }
                // (through the odd steps' exchange slots: step 0 writes the even ones right away)
                xch[2 * BM + wg * BM + row_l] = ss;
                asm volatile("bar.sync 1, 256;" ::: "memory");
                ss = __fadd_rn(xch[2 * BM + row_l], xch[3 * BM + row_l]);
                const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 256.0f), p.eps)));
                const uint4 *wq = reinterpret_cast<const uint4 *>(smem + OFF_WQ);
                const uint8_t *cs_row = smem + OFF_CS + row_l * 128;
#pragma unroll
                for (int c = 2 * wg; c < 2 * wg + 2; c++) {
                    float t[64];                                   // box c: dims 64c .. 64c+63, normed
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const uint4 x = *reinterpret_cast<const uint4 *>(q_row + c * IO_BOX + ((e ^ sw) << 4));
                        const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
                        const uint4 w4 = wq[c * 8 + e];
                        const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            float lo = __fmul_rn(__uint_as_float(xw[i] << 16), inv), hi = __fmul_rn(__uint_as_float(xw[i] & 0xffff0000u), inv);
                            if (p.q_norm_w) { lo = __fmul_rn(lo, __uint_as_float(ww[i] << 16)); hi = __fmul_rn(hi, __uint_as_float(ww[i] & 0xffff0000u)); }
                            t[e * 8 + 2 * i] = lo; t[e * 8 + 2 * i + 1] = hi;
                        }
                    }
                    if (c == 0) {
                        // pairs (d, d + 32), d < 32; cos in the first box of the row's table, sin in the second
#pragma unroll
                        for (int k = 0; k < 8; k++) {
                            const float4 cs = *reinterpret_cast<const float4 *>(cs_row + ((k ^ sw) << 4));
                            const float4 sn = *reinterpret_cast<const float4 *>(cs_row + IO_BOX + ((k ^ sw) << 4));
                            const float c4[4] = {cs.x, cs.y, cs.z, cs.w}, s4[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const int d = k * 4 + i;
                                const float lo = t[d], hi = t[d + 32];
                                t[d] = __fsub_rn(__fmul_rn(lo, c4[i]), __fmul_rn(hi, s4[i]));
                                t[d + 32] = __fadd_rn(__fmul_rn(hi, c4[i]), __fmul_rn(lo, s4[i]));
                            }
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 32; e++) v[e] = pack_bf16(t[2 * e], t[2 * e + 1]);
                    if (wg == 0) {
                        tmem_st32(t_q + lane_base + c * 32, v);
                    } else {
                        // dims 128-255: back to shared memory as the K-major swizzled operand
                        uint8_t *dst = smem + OFF_QHI + (c - 2) * IO_BOX + row_l * 128;
#pragma unroll
                        for (int e = 0; e < 8; e++)
                            *reinterpret_cast<uint4 *>(dst + ((e ^ sw) << 4)) = make_uint4(v[e * 4], v[e * 4 + 1], v[e * 4 + 2], v[e * 4 + 3]);
                    }
                }
                if (wg == 1) fence_proxy_async();            // those stores are read by the tensor core
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[Q_READY]);      // also releases the V stages to the TMA producer
        }
        // P in tensor memory: this thread's 64 keys of the step are 32 columns of bf16 pairs in its row's lane
        const uint32_t p_cols = t_p + lane_base + wg * 32;
        for (int j = 0; j < n_t; j++) {
            mbar_wait_hot(&bars[S_READY], j & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
            tc_fence_after();
            const int key0 = j * BN + wg * 64;
            // the row's 64 scores of this half, read once; S goes back to the tensor core at once
            uint32_t s0[32], s1[32];
            tmem_ld32(t_s + lane_base + wg * 64, s0);
            tmem_ld32(t_s + lane_base + wg * 64 + 32, s1);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[S_FREE]);
            if (key0 + 63 > p.base_pos + q0) {
#pragma unroll
                for (int e = 0; e < 32; e++) {
                    if (key0 + e > limit) s0[e] = __float_as_uint(NEG_BIG);
                    if (key0 + 32 + e > limit) s1[e] = __float_as_uint(NEG_BIG);
                }
            }
            float mxa = NEG_BIG, mxb = NEG_BIG;
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                mxa = fmaxf(mxa, fmaxf(__uint_as_float(s0[e]), __uint_as_float(s1[e])));
                mxb = fmaxf(mxb, fmaxf(__uint_as_float(s0[e + 1]), __uint_as_float(s1[e + 1])));
            }
            // the other half's maximum (slots alternate between steps: a slot is rewritten only
            // after the barrier of the step in between, which every reader has then passed)
            float *slot = xch + (j & 1) * 2 * BM;
            slot[wg * BM + row_l] = fmaxf(mxa, mxb);
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const float mx2 = fmaxf(fmaxf(fmaxf(mxa, mxb), slot[(wg ^ 1) * BM + row_l]) * sc2, NEG_BIG);
            const bool grow = j > 0 && mx2 - m > RESCALE_AT;
            const float alpha = grow ? ex2(m - mx2) : 1.0f;
            if (j == 0 || grow) m = mx2;
            // weights (masked scores are NEG_BIG: their weight underflows to exactly 0), packed in place
            float la = 0.0f, lb = 0.0f;
            auto weights = [&](uint32_t(&s)[32], float &acc) {
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const float x0 = ex2(fmaf(__uint_as_float(s[e]), sc2, -m));
                    const float x1 = ex2(fmaf(__uint_as_float(s[e + 1]), sc2, -m));
                    acc += x0 + x1;
                    s[e >> 1] = pack_bf16(x0, x1);      // slot e/2 <= e: already consumed
                }
            };
            // 16 packed pairs per 32 scores = 16 columns
            auto store_p = [&](const uint32_t(&s)[32], int col0) {
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 16; c++) pk[c] = s[c];
                tmem_st16(p_cols + col0, pk);
            };
            // All 64 weights are worked out (and packed in place) before this thread looks at the
            // tensor core again: P_{j-1} must have been consumed (and O be complete) before P is
            // overwritten or O rescaled, and P V of step j-1 ends about when these exponentials do;
            // what is left after that wait -- two stores into tensor memory -- is short, so the next
            // P V can be queued while Q K^T of the step after it still runs.
            weights(s0, la);
            weights(s1, lb);
            l = l * alpha + (la + lb);
            if (j > 0) {
                mbar_wait_hot(&bars[PV_DONE], (j - 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
                tc_fence_after();
            }
            if (__any_sync(0xffffffffu, grow)) {               // both halves of a row see the same flag
#pragma unroll 1
                for (int c = 4 * wg; c < 4 * wg + 4; c++) {
                    tmem_ld32(t_o + lane_base + c * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 32; e++) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                    tmem_st32(t_o + lane_base + c * 32, v);
                }
            }
            store_p(s0, 0);
            store_p(s1, 16);
            tmem_wait_st();               // the weights are in tensor memory before the P V issuer is told
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[P_READY]);
        }
        // the row's sum: both halves
        {
            float *slot = xch + (n_t & 1) * 2 * BM;
            slot[wg * BM + row_l] = l;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            l += slot[(wg ^ 1) * BM + row_l];
        }
        // epilogue: each 128-byte slice of the row (64 bf16 or 32 f32 outputs) is normalised,
        // multiplied by the sigmoid of the gate slice found at the same place of the gate tile,
        // written back over it, and the box is handed to the copy engine as soon as the four
        // warps of the half are through with it.  Rows past the end of the chunk are not written.
        mbar_wait_hot(&bars[PV_DONE], (n_t - 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
        tc_fence_after();
        if (p.gate) mbar_wait(&bars[G_FULL], 0, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        const bool gated = p.gate != nullptr;
        const bool elected = (warp & 3) == 0 && lane == 0;
        uint8_t *io_row = smem + OFF_STAGE_IO + row_l * 128;
        // o / l * sigmoid(g) with sigmoid(g) = 0.5 + 0.5 tanh(g / 2): one special-function operation per
        // element instead of two (an exponential and a reciprocal) -- the tile has 32 768 of them and
        // the unit delivers 16 per clock, which was a third of the time a CTA spends outside its main
        // loop.  tanh.approx is good to 2^-11, beside an output that is rounded to bf16 or held to 1e-2.
        const float half_inv = 0.5f * inv;
        auto sig = [&](float o, float g) {
            float t;
            asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * g));
            return o * fmaf(t, half_inv, half_inv);
        };
        auto publish = [&](int box, int x) {
            fence_proxy_async();
            if (wg == 0) asm volatile("bar.sync 2, 128;" ::: "memory");
            else asm volatile("bar.sync 3, 128;" ::: "memory");
            if (elected) {
                tma_store_2d(&p.omap, x, q0, smem + OFF_STAGE_IO + box * IO_BOX);
                tma_store_commit();
            }
        };
        if (p.out_dtype == DT_BF16) {
#pragma unroll 1
            for (int c = 4 * wg; c < 4 * wg + 4; c++) {        // 32 outputs = 64 bytes = half a box row
                tmem_ld32(t_o + lane_base + c * 32, v);
                tmem_wait_ld();
                uint8_t *bx = io_row + (c >> 1) * IO_BOX;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    uint4 *slot = reinterpret_cast<uint4 *>(bx + ((((c & 1) * 4 + k) ^ sw) << 4));
                    float o[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) o[e] = __uint_as_float(v[k * 8 + e]);
                    if (gated) {
                        const uint4 g = *slot;
                        const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            o[2 * e] = sig(o[2 * e], __uint_as_float(gw[e] << 16));
                            o[2 * e + 1] = sig(o[2 * e + 1], __uint_as_float(gw[e] & 0xffff0000u));
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; e++) o[e] *= inv;
                    }
                    *slot = make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
                }
                if (c & 1) publish(c >> 1, head * 256 + (c >> 1) * 64);
            }
        } else {
#pragma unroll 1
            for (int c = 4 * wg; c < 4 * wg + 4; c++) {        // 32 outputs = 128 bytes = one box row
                tmem_ld32(t_o + lane_base + c * 32, v);
                tmem_wait_ld();
                uint8_t *bx = io_row + c * IO_BOX;
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    float4 *slot = reinterpret_cast<float4 *>(bx + ((k ^ sw) << 4));
                    float4 o = make_float4(__uint_as_float(v[k * 4]), __uint_as_float(v[k * 4 + 1]),
                                           __uint_as_float(v[k * 4 + 2]), __uint_as_float(v[k * 4 + 3]));
                    if (gated) {
                        const float4 g = *slot;
                        o = make_float4(sig(o.x, g.x), sig(o.y, g.y), sig(o.z, g.z), sig(o.w, g.w));
                    } else {
                        o = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
                    }
                    *slot = o;
                }
                publish(c, head * 256 + c * 32);
            }
        }
        if (elected) tma_store_wait_read();                   // shared memory must outlive the copies
    }
    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace

bool attn_prefill_io_ok(const void *out, int out_dtype, const void *gate, int gate_dtype, int gate_stride) {
    const size_t el = out_dtype == DT_BF16 ? 2 : 4;
    if (reinterpret_cast<uintptr_t>(out) & 15) return false;
    if (!gate) return true;
    return gate_dtype == out_dtype && !(reinterpret_cast<uintptr_t>(gate) & 15) && gate_stride >= 256 && (gate_stride * el) % 16 == 0;
}

void launch_attn_prefill(cudaStream_t s, const PrefillParams &p) {
    static bool configured[64] = {false};      // the attribute is per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(qw_attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        configured[dev] = true;
    }
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = cudaLaunchConfig_t();
    cfg.gridDim = dim3((unsigned)(p.n_q_tiles * p.q_heads)); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM_BYTES; cfg.stream = s;
    cfg.attrs = &attr; cfg.numAttrs = g_tune_pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, qw_attn_prefill_kernel, p);
    g_launches++;
}

}  // namespace qw
