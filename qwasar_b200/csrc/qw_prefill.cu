// Causal prefill attention over the bf16 KV cache: tcgen05 tensor cores, accumulators in
// tensor memory, operands staged by TMA (sm_100a).
//
// One CTA per (128-row query tile, query head).  K and V are read from the cache (the rows
// of this chunk were appended just before), 64 keys -- one arena page -- per step, each
// double-buffered in shared memory:
//
//   warp 5   TMA: K tiles   (4 SWIZZLE_128B boxes of 64 keys x 64 dims each, 3 stages)
//   warp 6   TMA: V tiles   (likewise)
//   warp 4   one thread issues tcgen05.mma:  S_b = Q K_j^T   (TS, M128 N64  K16 x 16, Q in TMEM)
//                                            O  += P_j V_j   (TS, M128 N256 K16 x 4,  P in TMEM)
//   warps 0-3  softmax: thread i owns query row i = TMEM lane i.  Reads S (fp32) from TMEM,
//            online max / sum in the exp2 domain, writes P (bf16) back over S, rescales O in
//            TMEM only when a row's max grew by more than 2^8 (the stale max is exact
//            arithmetic, just a different common factor), and at the end normalises, applies
//            the sigmoid output gate and stores the row.
//
// TMEM columns (512): O [0,256) fp32 | Q [256,384) bf16 pairs | S0 [384,448) | S1 [448,512);
// P_b aliases the first 32 columns of S_b.  The query tile lives in tensor memory, not shared
// memory: as the A operand of every Q K^T it would otherwise be re-read from shared memory for
// each key tile (64 KB per 64 keys, as much as K and V together), and shared-memory bandwidth,
// not the tensor pipe, would bound the kernel.  Each softmax thread loads its own row of Q
// once and stores it to its TMEM lane.  S is double-buffered so that Q K_{j+1}^T runs under
// the softmax of tile j; K and V have three stages each so that loads run well ahead.
// Every wait on an mbarrier is bounded (qw_common.cuh): a stuck pipeline ends the kernel with
// a status code instead of hanging the GPU, and TMEM is always released.
//
// FLOPs per (row, key): 4 * 256 (QK^T and PV), the count of tools/bench/fabench.c:37-38.
#include "qw_kernels.h"

namespace qw {

namespace {

constexpr int BM = 128, BN = 64;
constexpr int NKV = 3;                                // shared-memory stages of K and of V
constexpr int KV_BYTES = BN * 512;                    // 64 keys x 256 dims bf16
constexpr int KVBOX = BN * 128;                       // one 64-dim box of a K or V tile
constexpr int OFF_K = 0, OFF_V = NKV * KV_BYTES, OFF_BAR = 2 * NKV * KV_BYTES;
constexpr int COL_O = 0, COL_Q = 256, COL_S = 384;    // TMEM columns
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
constexpr int THREADS = 7 * 32;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_BIG = -1.0e30f;
constexpr float RESCALE_AT = 8.0f;                    // log2 units

enum Bar { Q_READY = 0, K_FULL0, K_FULL1, K_FULL2, V_FULL0, V_FULL1, V_FULL2, K_FREE0, K_FREE1, K_FREE2,
           V_FREE0, V_FREE1, V_FREE2, S_READY0, S_READY1, P_READY0, P_READY1, PV_DONE, N_BARS };

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

__device__ __forceinline__ float load_gate(const void *g, size_t i, int dtype) {
    return dtype == DT_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(g)[i])
                            : reinterpret_cast<const float *>(g)[i];
}

__global__ void __launch_bounds__(THREADS, 1) qw_attn_prefill_kernel(const __grid_constant__ PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
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
        for (int i = 0; i < N_BARS; i++) mbar_init(&bars[i], (i == P_READY0 || i == P_READY1 || i == Q_READY) ? 128 : 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_o = tmem + COL_O, t_q = tmem + COL_Q, t_s0 = tmem + COL_S;

    if (warp == 5 || warp == 6) {
        // ---------------- warp 5: K tiles; warp 6: V tiles ----------------
        if (lane == 0) {
            const bool is_k = warp == 5;
            const KvLayer &L = is_k ? p.kc : p.vc;
            const CUtensorMap *map = is_k ? &p.kmap : &p.vmap;
            const int FULL = is_k ? K_FULL0 : V_FULL0, FREE = is_k ? K_FREE0 : V_FREE0;
            uint8_t *base = smem + (is_k ? OFF_K : OFF_V);
            for (int j = 0; j < n_t; j++) {
                const int st = j % NKV;
                const int t = j * BN;
                int64_t row;
                if (L.table) {
                    const int pg = j < L.pt_stride ? __ldg(L.table + (size_t)kvh * L.pt_stride + j) : -1;
                    row = pg >= 0 ? (int64_t)pg * QW_PAGE_TOKENS : (int64_t)p.oob_row;   // unmapped: zero fill
                } else {
                    row = t < L.max_ctx ? (int64_t)kvh * L.max_ctx + t : (int64_t)p.oob_row;
                }
                if (j >= NKV) mbar_wait(&bars[FREE + st], ((j / NKV) - 1) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
                mbar_expect_tx(&bars[FULL + st], KV_BYTES);
#pragma unroll
                for (int b = 0; b < 4; b++)
                    tma_load_2d(base + st * KV_BYTES + b * KVBOX, map, b * 64, (int32_t)row, &bars[FULL + st]);
            }
        }
    } else if (warp == 4) {
        // ---------------- tensor-core issue ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc(128, BN, 0);
            constexpr uint32_t idesc_pv = instr_desc(128, 256, 1);
            const uint32_t k_a = smem_u32(smem + OFF_K), v_a = smem_u32(smem + OFF_V);
            constexpr uint32_t hi = desc_hi(1024);
            auto issue_qk = [&](int j) {
                const int st = j % NKV;
                mbar_wait(&bars[K_FULL0 + st], (j / NKV) & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                tc_fence_after();
                const uint32_t t_s = t_s0 + (j & 1) * BN;
                const uint32_t k_lo = desc_lo(k_a + st * KV_BYTES, 16);
                // A: 16 dims of Q = 8 TMEM columns; B: 16 dims = 32 bytes (2 units) inside the swizzle atom,
                // 64 dims per box (KVBOX / 16 units)
                mma_ts<false>(t_s, t_q, k_lo, hi, idesc_qk);
#pragma unroll
                for (int ks = 1; ks < 16; ks++)
                    mma_ts<true>(t_s, t_q + ks * 8, k_lo + (ks >> 2) * (KVBOX >> 4) + (ks & 3) * 2, hi, idesc_qk);
                tc_commit(&bars[S_READY0 + (j & 1)]);
                tc_commit(&bars[K_FREE0 + st]);
            };
            mbar_wait(&bars[Q_READY], 0, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
            issue_qk(0);
            for (int j = 0; j < n_t; j++) {
                const int st = j % NKV;
                if (j + 1 < n_t) issue_qk(j + 1);
                mbar_wait(&bars[P_READY0 + (j & 1)], (j >> 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
                mbar_wait(&bars[V_FULL0 + st], (j / NKV) & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                tc_fence_after();
                const uint32_t t_p = t_s0 + (j & 1) * BN;      // P aliases the head of S
                const uint32_t v_lo = desc_lo(v_a + st * KV_BYTES, KVBOX);
                // 16 keys per step: 8 TMEM columns of bf16 pairs, 2048 bytes (128 units) of V
                if (j > 0) mma_ts<true>(t_o, t_p, v_lo, hi, idesc_pv);
                else mma_ts<false>(t_o, t_p, v_lo, hi, idesc_pv);
#pragma unroll
                for (int ks = 1; ks < BN / 16; ks++) mma_ts<true>(t_o, t_p + ks * 8, v_lo + ks * 128, hi, idesc_pv);
                tc_commit(&bars[PV_DONE]);
                tc_commit(&bars[V_FREE0 + st]);
            }
        }
    } else {
        // ---------------- softmax + epilogue: thread = query row = TMEM lane ----------------
        const int row_l = warp * 32 + lane;
        const int row_g = q0 + row_l;
        const bool valid = row_g < p.rows;
        const int limit = valid ? p.base_pos + row_g : 0x7fffffff;         // last key this row may read
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float sc2 = p.scale * LOG2E;
        float m = NEG_BIG, l = 0.0f;
        uint32_t v[32];
        {
            // this row of Q (256 bf16 = 128 columns of pairs) into the row's TMEM lane
            const uint4 *src = reinterpret_cast<const uint4 *>(p.q + ((size_t)row_g * p.q_heads + head) * 256);
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const uint4 x = valid ? __ldg(src + c * 8 + e) : make_uint4(0, 0, 0, 0);
                    v[e * 4] = x.x; v[e * 4 + 1] = x.y; v[e * 4 + 2] = x.z; v[e * 4 + 3] = x.w;
                }
                tmem_st32(t_q + lane_base + c * 32, v);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars[Q_READY]);
        }
        for (int j = 0; j < n_t; j++) {
            const uint32_t t_s = t_s0 + (j & 1) * BN + lane_base;
            mbar_wait(&bars[S_READY0 + (j & 1)], (j >> 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
            tc_fence_after();
            const bool need_mask = j * BN + BN - 1 > p.base_pos + q0;
            // the row's 64 scores, read once
            uint32_t sa[32], sb[32];
            tmem_ld32(t_s, sa);
            tmem_ld32(t_s + 32, sb);
            tmem_wait_ld();
            if (need_mask) {
#pragma unroll
                for (int e = 0; e < 32; e++) {
                    if (j * BN + e > limit) sa[e] = __float_as_uint(NEG_BIG);
                    if (j * BN + 32 + e > limit) sb[e] = __float_as_uint(NEG_BIG);
                }
            }
            float mx = NEG_BIG;
#pragma unroll
            for (int e = 0; e < 32; e++) mx = fmaxf(mx, fmaxf(__uint_as_float(sa[e]), __uint_as_float(sb[e])));
            const float mx2 = fmaxf(mx * sc2, NEG_BIG);
            if (j == 0) {
                m = mx2;
            } else {
                const bool grow = mx2 - m > RESCALE_AT;
                if (__any_sync(0xffffffffu, grow)) {
                    // O must hold every product issued so far before it is rescaled
                    mbar_wait(&bars[PV_DONE], (j - 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
                    tc_fence_after();
                    const float alpha = grow ? ex2(m - mx2) : 1.0f;
#pragma unroll 1
                    for (int c = 0; c < 8; c++) {
                        tmem_ld32(t_o + lane_base + c * 32, v);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; e++) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                        tmem_st32(t_o + lane_base + c * 32, v);
                    }
                    tmem_wait_st();
                    l *= alpha;
                    if (grow) m = mx2;
                }
            }
            // weights, their sum, and P (bf16) written over the head of S; masked scores are
            // NEG_BIG, whose weight underflows to exactly 0
            uint32_t pk[32];
            float l0 = 0.0f, l1 = 0.0f;
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                const float x0 = ex2(fmaf(__uint_as_float(sa[e]), sc2, -m));
                const float x1 = ex2(fmaf(__uint_as_float(sa[e + 1]), sc2, -m));
                const float y0 = ex2(fmaf(__uint_as_float(sb[e]), sc2, -m));
                const float y1 = ex2(fmaf(__uint_as_float(sb[e + 1]), sc2, -m));
                l0 += x0 + x1;
                l1 += y0 + y1;
                pk[e >> 1] = pack_bf16(x0, x1);
                pk[16 + (e >> 1)] = pack_bf16(y0, y1);
            }
            l += l0 + l1;
            tmem_st32(t_s, pk);
            tmem_wait_st();
            // Observe every phase of PV_DONE: a parity wait is only meaningful for a waiter at most
            // one phase behind, and the epilogue (or a later rescale) waits on this barrier again.
            // P V_{j-1} was issued long before this point, and P V_j cannot be issued until every
            // row has arrived below, so the barrier cannot run ahead of this wait.
            if (j > 0) mbar_wait(&bars[PV_DONE], (j - 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
            tc_fence_before();
            mbar_arrive(&bars[P_READY0 + (j & 1)]);
        }
        // epilogue
        mbar_wait(&bars[PV_DONE], (n_t - 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
        tc_fence_after();
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        const size_t rh = (size_t)row_g * p.q_heads + head;
#pragma unroll 1
        for (int c = 0; c < 8; c++) {
            tmem_ld32(t_o + lane_base + c * 32, v);
            tmem_wait_ld();
            if (valid) {
                float o[32];
#pragma unroll
                for (int e = 0; e < 32; e++) o[e] = __uint_as_float(v[e]) * inv;
                if (p.gate) {
                    const size_t gi = rh * p.gate_stride + c * 32;
#pragma unroll
                    for (int e = 0; e < 32; e++) o[e] *= 1.0f / (1.0f + __expf(-load_gate(p.gate, gi + e, p.gate_dtype)));
                }
                if (p.out_dtype == DT_BF16) {
                    uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(p.out) + rh * 256 + c * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++)
                        dst[q4] = make_uint4(pack_bf16(o[q4 * 8], o[q4 * 8 + 1]), pack_bf16(o[q4 * 8 + 2], o[q4 * 8 + 3]),
                                             pack_bf16(o[q4 * 8 + 4], o[q4 * 8 + 5]), pack_bf16(o[q4 * 8 + 6], o[q4 * 8 + 7]));
                } else {
                    float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + rh * 256 + c * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 8; q4++) dst[q4] = make_float4(o[q4 * 4], o[q4 * 4 + 1], o[q4 * 4 + 2], o[q4 * 4 + 3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace

void launch_attn_prefill(cudaStream_t s, const PrefillParams &p) {
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(qw_attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        configured = true;
    }
    qw_attn_prefill_kernel<<<p.n_q_tiles * p.q_heads, THREADS, SMEM_BYTES, s>>>(p);
    g_launches++;
}

}  // namespace qw
