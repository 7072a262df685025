// Causal prefill attention, CTA-pair version: two CTAs of a thread-block cluster (the two query
// heads 2u, 2u+1 of one 128-row tile, which share a kv head) drive the tensor cores as one
// `cta_group::2` unit with M = 256.
//
// Why pairs: tensor memory holds one 128-row accumulator per CTA at head_dim 256 (O alone is 256
// of the 512 columns), so a lone CTA re-reads every K/V tile from L2 for just 128 rows -- 128
// FLOP per L2 byte -- and the L2 -> SM stream, not the tensor pipe, sets the pace.  In a pair
// each CTA loads only half of every tile (CTA r: keys [64r, 64r+64) of the 128-key K tile, dims
// [128r, 128r+128) of the V tile) and the pair's MMA reads both halves, so the same stream feeds
// twice the rows; the halved stages also leave room for three K and three V stages.
//
// Everything else follows qw_prefill.cu: Q in tensor memory as the A operand of Q K^T, S read
// into registers and handed back at once, P through shared memory as the A operand of P V, lazy
// rescale of O, prologue/epilogue staged through shared memory.  CTA 0 (the leader) issues every
// tcgen05.mma; TMA loads of both CTAs signal the leader's "full" barriers (`.cta_group::2` loads,
// no multicast); tcgen05.commit multicasts "free"/"ready" arrivals to both CTAs; the softmax
// threads of both CTAs arrive on the leader's barriers through cluster shared-memory addresses.
// Every wait is bounded and the kernel always releases its tensor memory.
#include "qw_kernels.h"

namespace qw {

namespace {

constexpr int BM = 128, BN = 128;                     // query rows per CTA, keys per step
constexpr int NKV = 3;                                // stages of K and of V
constexpr int K_BYTES = 64 * 512;                     // this CTA's half of a K tile: 64 keys x 256 dims
constexpr int KBOX = 64 * 128;                        // one 64-dim box of it
constexpr int V_BYTES = BN * 256;                     // this CTA's half of a V tile: 128 keys x 128 dims
constexpr int VBOX = BN * 128;                        // one 64-dim box of it (128 keys)
constexpr int P_BYTES = BM * BN * 2;
constexpr int PBOX = BM * 128;
constexpr int OFF_K = 0, OFF_V = NKV * K_BYTES, OFF_P = OFF_V + NKV * V_BYTES, OFF_BAR = OFF_P + P_BYTES;
constexpr int OFF_STAGE_O = OFF_K;                    // the normalised O tile (fp32, 1040-byte rows) over the idle K/V stages
constexpr int COL_O = 0, COL_Q = 256, COL_S = 384;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB a CTA may use");
constexpr int THREADS = 7 * 32;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_BIG = -1.0e30f;
constexpr float RESCALE_AT = 8.0f;

// K_FULL / V_FULL / Q_READY / S_FREE / P_READY are waited on by the leader only (arrivals and TMA
// bytes come from both CTAs); the others exist in both CTAs and are signalled by multicast commits.
enum Bar { Q_READY = 0, Q_STAGED, K_FULL0, K_FULL1, K_FULL2, V_FULL0, V_FULL1, V_FULL2, K_FREE0, K_FREE1, K_FREE2,
           V_FREE0, V_FREE1, V_FREE2, S_READY, S_FREE, P_READY, PV_DONE, N_BARS };

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_cta(uint64_t *bar, uint32_t rank) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(smem_u32(bar)), "r"(rank) : "memory");
}

// ---- tcgen05, cta_group::2 -------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc2(uint32_t *slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// arrival on the same barrier of both CTAs once all earlier tcgen05 operations have completed
__device__ __forceinline__ void tc_commit2(uint64_t *bar) {
    asm volatile(
        "{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
        ::"r"(smem_u32(bar)) : "memory");
}
template <bool ACC>
__device__ __forceinline__ void mma2_ts(uint32_t d, uint32_t a_tmem, uint32_t bdesc_lo, uint32_t bdesc_hi, uint32_t idesc) {
    if (ACC)
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\tsetp.eq.u32 p, 0, 0;\n\tmov.b64 bd, {%2, %3};\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], bd, %4, p;\n\t}"
            ::"r"(d), "r"(a_tmem), "r"(bdesc_lo), "r"(bdesc_hi), "r"(idesc) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\tsetp.ne.u32 p, 0, 0;\n\tmov.b64 bd, {%2, %3};\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], bd, %4, p;\n\t}"
            ::"r"(d), "r"(a_tmem), "r"(bdesc_lo), "r"(bdesc_hi), "r"(idesc) : "memory");
}
template <bool ACC>
__device__ __forceinline__ void mma2_ss(uint32_t d, uint32_t adesc_lo, uint32_t adesc_hi, uint32_t bdesc_lo, uint32_t bdesc_hi,
                                        uint32_t idesc) {
    if (ACC)
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 ad, bd;\n\tsetp.eq.u32 p, 0, 0;\n\tmov.b64 ad, {%1, %2};\n\tmov.b64 bd, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], ad, bd, %5, p;\n\t}"
            ::"r"(d), "r"(adesc_lo), "r"(adesc_hi), "r"(bdesc_lo), "r"(bdesc_hi), "r"(idesc) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 ad, bd;\n\tsetp.ne.u32 p, 0, 0;\n\tmov.b64 ad, {%1, %2};\n\tmov.b64 bd, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], ad, bd, %5, p;\n\t}"
            ::"r"(d), "r"(adesc_lo), "r"(adesc_hi), "r"(bdesc_lo), "r"(bdesc_hi), "r"(idesc) : "memory");
}
// TMA load whose bytes are counted on the LEADER's barrier (same offset, CTA-rank bit cleared).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *map, int32_t x, int32_t y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar) & 0xFEFFFFFFu) : "memory");
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
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
    return ((addr >> 4) & 0x3FFF) | (((lbo_bytes >> 4) & 0x3FFF) << 16);
}
__device__ __forceinline__ constexpr uint32_t desc_hi(uint32_t sbo_bytes) {
    return ((sbo_bytes >> 4) & 0x3FFF) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ constexpr uint32_t instr_desc(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
qw_attn_prefill_pair_kernel(const __grid_constant__ PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    // identical offsets in both CTAs are required: the dynamic segment starts at the same address in each
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + OFF_BAR);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + N_BARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();               // 0 = leader
    const int qt = p.n_q_tiles - 1 - (int)(blockIdx.x / p.q_heads);
    const int head = blockIdx.x % p.q_heads;             // the pair: heads 2u (leader) and 2u+1, same kv head
    const int kvh = head / p.gqa;
    const int q0 = qt * BM;
    const int n_keys = p.base_pos + p.rows;
    const int k_end = min(n_keys, p.base_pos + q0 + BM);
    const int n_t = (k_end + BN - 1) / BN;

    if (threadIdx.x == 0) {
        for (int i = 0; i < N_BARS; i++) {
            uint32_t cnt = 1;
            if (i == Q_READY || i == S_FREE || i == P_READY) cnt = 8;       // one per softmax warp, both CTAs
            if (i == Q_STAGED) cnt = 4;
            mbar_init(&bars[i], cnt);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) tmem_alloc2(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                      // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_o = tmem + COL_O, t_q = tmem + COL_Q, t_s = tmem + COL_S;

    auto page_row = [&](const KvLayer &L, int pg) -> int32_t {
        if (L.table) {
            const int id = pg < L.pt_stride ? __ldg(L.table + (size_t)kvh * L.pt_stride + pg) : -1;
            return id >= 0 ? id * QW_PAGE_TOKENS : p.oob_row;
        }
        return pg * QW_PAGE_TOKENS < L.max_ctx ? kvh * L.max_ctx + pg * QW_PAGE_TOKENS : p.oob_row;
    };

    if ((warp == 5 || warp == 6) && lane > 0 && p.gate) {
        // idle lanes: pull this tile's gate rows into L2 while the main loop runs (the epilogue reads them)
        const size_t el = p.gate_dtype == DT_BF16 ? 2 : 4;
        const int n_valid = min(BM, p.rows - q0);
        const int lines = (int)(256 * el / 128);
        for (int i = (warp - 5) * 31 + lane - 1; i < n_valid * lines; i += 62) {
            const int r = i / lines, ln = i - r * lines;
            const char *a = reinterpret_cast<const char *>(p.gate) + (((size_t)(q0 + r) * p.q_heads + head) * p.gate_stride) * el + ln * 128;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
        }
    }
    if (warp == 5) {
        // ---------------- K: this CTA's 64 keys (one page) of every 128-key tile ----------------
        if (lane == 0) {
            mbar_wait(&bars[Q_STAGED], 0, abort_flag, p.status, QW_ST_MMA_TIMEOUT);   // the Q staging borrowed this region
            for (int j = 0; j < n_t; j++) {
                const int st = j % NKV;
                const int32_t r = page_row(p.kc, 2 * j + (int)rank);
                if (j >= NKV) mbar_wait(&bars[K_FREE0 + st], ((j / NKV) - 1) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
                if (rank == 0) mbar_expect_tx(&bars[K_FULL0 + st], 2 * K_BYTES);       // both CTAs' bytes land on this barrier
#pragma unroll
                for (int b = 0; b < 4; b++)
                    tma_load_2d_pair(smem + OFF_K + st * K_BYTES + b * KBOX, &p.kmap, b * 64, r, &bars[K_FULL0 + st]);
            }
        }
    } else if (warp == 6) {
        // ---------------- V: this CTA's 128 dims of every 128-key tile (two pages) ----------------
        if (lane == 0) {
            for (int j = 0; j < n_t; j++) {
                const int st = j % NKV;
                const int32_t r0 = page_row(p.vc, 2 * j), r1 = page_row(p.vc, 2 * j + 1);
                if (j >= NKV) mbar_wait(&bars[V_FREE0 + st], ((j / NKV) - 1) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
                if (rank == 0) mbar_expect_tx(&bars[V_FULL0 + st], 2 * V_BYTES);
                uint8_t *dst = smem + OFF_V + st * V_BYTES;
#pragma unroll
                for (int b = 0; b < 2; b++) {
                    const int x = ((int)rank * 2 + b) * 64;
                    tma_load_2d_pair(dst + b * VBOX, &p.vmap, x, r0, &bars[V_FULL0 + st]);
                    tma_load_2d_pair(dst + b * VBOX + 8192, &p.vmap, x, r1, &bars[V_FULL0 + st]);
                }
            }
        }
    } else if (warp == 4) {
        // ---------------- tensor-core issue: the leader drives both CTAs ----------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc_qk = instr_desc(256, BN, 0);
            constexpr uint32_t idesc_pv = instr_desc(256, 256, 1);
            constexpr uint32_t hi = desc_hi(1024);
            const uint32_t k_a = smem_u32(smem + OFF_K), v_a = smem_u32(smem + OFF_V), p_a = smem_u32(smem + OFF_P);
            const uint32_t p_lo = desc_lo(p_a, 16);
            auto issue_qk = [&](int j) {
                const int st = j % NKV;
                mbar_wait(&bars[K_FULL0 + st], (j / NKV) & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                tc_fence_after();
                const uint32_t k_lo = desc_lo(k_a + st * K_BYTES, 16);
                mma2_ts<false>(t_s, t_q, k_lo, hi, idesc_qk);
#pragma unroll
                for (int ks = 1; ks < 16; ks++)
                    mma2_ts<true>(t_s, t_q + ks * 8, k_lo + (ks >> 2) * (KBOX >> 4) + (ks & 3) * 2, hi, idesc_qk);
                tc_commit2(&bars[S_READY]);
                tc_commit2(&bars[K_FREE0 + st]);
            };
            mbar_wait(&bars[Q_READY], 0, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
            issue_qk(0);
            for (int j = 0; j < n_t; j++) {
                const int st = j % NKV;
                if (j + 1 < n_t) {
                    mbar_wait(&bars[S_FREE], j & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
                    issue_qk(j + 1);
                }
                mbar_wait(&bars[P_READY], j & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
                mbar_wait(&bars[V_FULL0 + st], (j / NKV) & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                tc_fence_after();
                const uint32_t v_lo = desc_lo(v_a + st * V_BYTES, VBOX);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    // A: 16 keys of P = 32 bytes inside the swizzle atom, 64 keys per box; B: 16 keys of V = 2048 bytes
                    const uint32_t a_lo = p_lo + (ks >> 2) * (PBOX >> 4) + (ks & 3) * 2;
                    if (j > 0 || ks > 0) mma2_ss<true>(t_o, a_lo, hi, v_lo + ks * 128, hi, idesc_pv);
                    else mma2_ss<false>(t_o, a_lo, hi, v_lo + ks * 128, hi, idesc_pv);
                }
                tc_commit2(&bars[PV_DONE]);
                tc_commit2(&bars[V_FREE0 + st]);
            }
        }
    } else {
        // ---------------- softmax + epilogue: thread = query row = TMEM lane ----------------
        const int row_l = warp * 32 + lane;
        const int row_g = q0 + row_l;
        const bool valid = row_g < p.rows;
        const int limit = valid ? p.base_pos + row_g : 0x7fffffff;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float sc2 = p.scale * LOG2E;
        float m = NEG_BIG, l = 0.0f;
        uint32_t v[32];
        {
            uint8_t *stage = smem + OFF_K;
            const uint4 *qsrc = reinterpret_cast<const uint4 *>(p.q);
#pragma unroll 16
            for (int k = 0; k < 32; k++) {
                const int idx = row_l + 128 * k, r = idx >> 5, ch = idx & 31;
                uint4 x = make_uint4(0, 0, 0, 0);
                if (q0 + r < p.rows) x = __ldg(qsrc + ((size_t)(q0 + r) * p.q_heads + head) * 32 + ch);
                *reinterpret_cast<uint4 *>(stage + r * 528 + ch * 16) = x;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const uint4 x = *reinterpret_cast<const uint4 *>(stage + row_l * 528 + (c * 8 + e) * 16);
                    v[e * 4] = x.x; v[e * 4 + 1] = x.y; v[e * 4 + 2] = x.z; v[e * 4 + 3] = x.w;
                }
                tmem_st32(t_q + lane_base + c * 32, v);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars[Q_STAGED]);             // this CTA's K region is free for its TMA producer
                mbar_arrive_cta(&bars[Q_READY], 0);       // the leader may start once both tiles are in tensor memory
            }
        }
        uint8_t *p_row = smem + OFF_P + row_l * 128;
        const uint32_t sw = row_l & 7;
        for (int j = 0; j < n_t; j++) {
            mbar_wait(&bars[S_READY], j & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
            tc_fence_after();
            const bool need_mask = j * BN + BN - 1 > p.base_pos + q0;
            uint32_t s0[32], s1[32], s2[32], s3[32];
            tmem_ld32(t_s + lane_base, s0);
            tmem_ld32(t_s + lane_base + 32, s1);
            tmem_ld32(t_s + lane_base + 64, s2);
            tmem_ld32(t_s + lane_base + 96, s3);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cta(&bars[S_FREE], 0);
            if (need_mask) {
#pragma unroll
                for (int e = 0; e < 32; e++) {
                    if (j * BN + e > limit) s0[e] = __float_as_uint(NEG_BIG);
                    if (j * BN + 32 + e > limit) s1[e] = __float_as_uint(NEG_BIG);
                    if (j * BN + 64 + e > limit) s2[e] = __float_as_uint(NEG_BIG);
                    if (j * BN + 96 + e > limit) s3[e] = __float_as_uint(NEG_BIG);
                }
            }
            float mxa = NEG_BIG, mxb = NEG_BIG;
#pragma unroll
            for (int e = 0; e < 32; e++) {
                mxa = fmaxf(mxa, fmaxf(__uint_as_float(s0[e]), __uint_as_float(s1[e])));
                mxb = fmaxf(mxb, fmaxf(__uint_as_float(s2[e]), __uint_as_float(s3[e])));
            }
            const float mx2 = fmaxf(fmaxf(mxa, mxb) * sc2, NEG_BIG);
            const bool grow = j > 0 && mx2 - m > RESCALE_AT;
            const float alpha = grow ? ex2(m - mx2) : 1.0f;
            if (j == 0 || grow) m = mx2;
            float la = 0.0f, lb = 0.0f;
            auto weights = [&](uint32_t(&s)[32], float &acc) {
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const float x0 = ex2(fmaf(__uint_as_float(s[e]), sc2, -m));
                    const float x1 = ex2(fmaf(__uint_as_float(s[e + 1]), sc2, -m));
                    acc += x0 + x1;
                    s[e >> 1] = pack_bf16(x0, x1);
                }
            };
            weights(s0, la); weights(s1, lb); weights(s2, la); weights(s3, lb);
            l = l * alpha + (la + lb);
            if (j > 0) {
                mbar_wait(&bars[PV_DONE], (j - 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
                tc_fence_after();
            }
            if (__any_sync(0xffffffffu, grow)) {
#pragma unroll 1
                for (int c = 0; c < 8; c++) {
                    tmem_ld32(t_o + lane_base + c * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 32; e++) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                    tmem_st32(t_o + lane_base + c * 32, v);
                }
                tmem_wait_st();
            }
            auto store_p = [&](const uint32_t(&s)[32], int box, int chunk0) {
#pragma unroll
                for (int c = 0; c < 4; c++)
                    *reinterpret_cast<uint4 *>(p_row + box * PBOX + (((chunk0 + c) ^ sw) << 4)) =
                        make_uint4(s[c * 4], s[c * 4 + 1], s[c * 4 + 2], s[c * 4 + 3]);
            };
            store_p(s0, 0, 0); store_p(s1, 0, 4); store_p(s2, 1, 0); store_p(s3, 1, 4);
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cta(&bars[P_READY], 0);
        }
        const int n_valid = min(BM, p.rows - q0);
        const int d2 = row_l * 2;
        constexpr int NB = 16;
        float ga0[NB], ga1[NB], gb0[NB], gb1[NB];     // two batches of gates: one in flight, one in use
        auto load_gates = [&](int r0, float(&g0)[NB], float(&g1)[NB]) {
            if (!p.gate) return;
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const int r = min(r0 + i, n_valid - 1);
                const size_t gi = ((size_t)(q0 + r) * p.q_heads + head) * p.gate_stride + d2;
                if (p.gate_dtype == DT_BF16) {
                    const __nv_bfloat162 g = __ldg(reinterpret_cast<const __nv_bfloat162 *>(reinterpret_cast<const __nv_bfloat16 *>(p.gate) + gi));
                    g0[i] = __low2float(g); g1[i] = __high2float(g);
                } else {
                    const float2 g = __ldg(reinterpret_cast<const float2 *>(reinterpret_cast<const float *>(p.gate) + gi));
                    g0[i] = g.x; g1[i] = g.y;
                }
            }
        };
        // The rows of a batch are read from shared memory first, all together: a shared-memory
        // load cannot be moved above the global store of the row before it (the compiler sees
        // two generic pointers), so a load-compute-store loop runs one row at a time.
        auto store_rows = [&](int r0, const float(&g0)[NB], const float(&g1)[NB]) {
            float2 o[NB];
#pragma unroll
            for (int i = 0; i < NB; i++)
                o[i] = *reinterpret_cast<const float2 *>(smem + OFF_STAGE_O + (size_t)min(r0 + i, n_valid - 1) * 1040 + d2 * 4);
            if (p.gate) {
#pragma unroll
                for (int i = 0; i < NB; i++) {
                    o[i].x = __fdividef(o[i].x, 1.0f + __expf(-g0[i]));
                    o[i].y = __fdividef(o[i].y, 1.0f + __expf(-g1[i]));
                }
            }
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const int r = r0 + i;
                if (r < n_valid) {
                    const size_t rh = (size_t)(q0 + r) * p.q_heads + head;
                    if (p.out_dtype == DT_BF16)
                        *reinterpret_cast<uint32_t *>(reinterpret_cast<__nv_bfloat16 *>(p.out) + rh * 256 + d2) = pack_bf16(o[i].x, o[i].y);
                    else
                        *reinterpret_cast<float2 *>(reinterpret_cast<float *>(p.out) + rh * 256 + d2) = o[i];
                }
            }
        };
        load_gates(0, ga0, ga1);
        mbar_wait(&bars[PV_DONE], (n_t - 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
        tc_fence_after();
        {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            float *orow = reinterpret_cast<float *>(smem + OFF_STAGE_O + (size_t)row_l * 1040);
#pragma unroll 1
            for (int c = 0; c < 8; c++) {
                tmem_ld32(t_o + lane_base + c * 32, v);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; e += 4)
                    *reinterpret_cast<float4 *>(orow + c * 32 + e) =
                        make_float4(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv,
                                    __uint_as_float(v[e + 2]) * inv, __uint_as_float(v[e + 3]) * inv);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            // the next batch's loads are issued before the current batch is consumed
#pragma unroll 1
            for (int r0 = 0; r0 < n_valid; r0 += 2 * NB) {
                if (r0 + NB < n_valid) load_gates(r0 + NB, gb0, gb1);
                store_rows(r0, ga0, ga1);
                if (r0 + 2 * NB < n_valid) load_gates(r0 + 2 * NB, ga0, ga1);
                if (r0 + NB < n_valid) store_rows(r0 + NB, gb0, gb1);
            }
        }
    }
    // neither CTA may leave while the pair's tensor cores can still read its shared or tensor memory
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc2(tmem, 512);
    }
}

}  // namespace

bool attn_prefill_pair_ok(const PrefillParams &p) { return p.gqa % 2 == 0 && p.q_heads % 2 == 0; }

void launch_attn_prefill_pair(cudaStream_t s, const PrefillParams &p) {
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(qw_attn_prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        configured[dev] = true;
    }
    qw_attn_prefill_pair_kernel<<<p.n_q_tiles * p.q_heads, THREADS, SMEM_BYTES, s>>>(p);
    g_launches++;
}

}  // namespace qw
