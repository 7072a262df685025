// Decode / speculative-verify attention over the bf16 KV cache (sm_100a).
//
// qw_attn_split_kernel -- the split-KV kernel.  All (sequence, kv head) groups of a
// launch are laid end to end as one line of 32-key tiles, and that line is cut into
// one equal share per CTA (one CTA per SM), so every SM streams the same number of
// bytes whatever the batch, head count or depth.  A share that crosses a group
// boundary is processed as two segments.  Per CTA:
//   * one producer warp walks the share and issues TMA loads (SWIZZLE_128B boxes of
//     32 keys x 64 dims) of K and V into a ring of 32 KB stages, mbarrier-tracked;
//   * MT x KG consumer warps: warp (mt, kg) owns query rows [16 mt, 16 mt + 16) of
//     the group (row i = r * gqa + g: all query heads of the kv head, all rows) and
//     every KG-th 16-key block; S = Q K^T and O += P V run on m16n8k16 bf16 tensor
//     ops with fp32 accumulators, the softmax is online in fp32 (exp2 domain), quad
//     reductions by shuffle;
//   * at a segment's end the warps' (m, l, O) are merged through shared memory and
//     written either as the final gated output (the segment was the whole group) or
//     as one partial (max, sum, un-normalised acc) per row.
// qw_attn_merge_kernel combines a group's partials by log-sum-exp and applies the
// sigmoid output gate, the arithmetic of the reference's qw_attn_merge_gated
// (metal/attn.metal:273-331).
//
// Bytes moved per key: 512 B of K + 512 B of V, once (the algorithmic minimum);
// partials add (n_cta + groups) x rows x 1 KB.
#include "qw_kernels.h"
#include <algorithm>
#include <cooperative_groups.h>

namespace qw {

namespace {

constexpr int TILE_KEYS = 32;
constexpr int STAGE_BYTES = TILE_KEYS * 512 * 2;          // K then V
constexpr int BOX_BYTES = TILE_KEYS * 128;                // 32 keys x 64 dims bf16
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float NEG_BIG = -1.0e30f;
constexpr int RED_LD = 264;        // floats per row of the reduction buffer: 8 of padding spread the rows over the banks

template <int MT, int KG_>
struct SplitCfg {
    static constexpr int KG = KG_;
    static constexpr int NW = MT * KG;                    // consumer warps
    static constexpr int NST = (MT == 1) ? 6 : (MT == 2 ? (KG_ == 3 ? 3 : 5) : 3);
    static constexpr int THREADS = (NW + 1) * 32;         // + the TMA producer warp
    static_assert(THREADS <= 256, "warps are allocated in fours: 9 warps would be budgeted as 12");
    // a warp must take part in every phase of each stage it ever waits on (a parity wait is only
    // valid one phase behind): the block -> warp pattern has to repeat with the ring
    static_assert((2 * NST) % KG == 0, "key groups must divide the blocks of one trip round the ring");
    static constexpr int MAXREG = 255;
    static constexpr int Q_BYTES = MT * 16 * 512;
    static constexpr int RED_BYTES = MT * 16 * RED_LD * 4;
    static constexpr int OFF_Q = NST * STAGE_BYTES;
    static constexpr int OFF_RED = OFF_Q + Q_BYTES;
    static constexpr int OFF_M = OFF_RED + RED_BYTES;     // [MT][KG][16] floats
    static constexpr int OFF_L = OFF_M + MT * KG * 16 * 4;  // [MT][16] floats
    static constexpr int OFF_BAR = OFF_L + MT * 16 * 4;   // full[NST], empty[NST], abort
    static constexpr int SMEM = OFF_BAR + (2 * NST + 1) * 8 + 1024;  // + alignment slack
    static_assert(SMEM <= 232448, "exceeds the 227 KB a CTA may use");
};

struct Cursor {      // position on the flattened tile line
    int s, h, t;     // sequence, kv head, tile within the group
};

__device__ __forceinline__ Cursor locate(const AttnParams &p, int T) {
    Cursor c;
    // the last sequence that starts at or before T, by bisection (every probe is an indexed read of the launch's
    // table: a walk over 64 sequences at the head of every warp cost the kernel 10 us)
    int s = 0, e = p.n_seq - 1;
    while (s < e) {
        const int m = (s + e + 1) >> 1;
        if (p.seq[m].cum_tiles <= T) s = m; else e = m - 1;
    }
    const int rel = T - p.seq[s].cum_tiles;
    c.s = s;
    c.h = rel / p.seq[s].n_tiles;
    c.t = rel - c.h * p.seq[s].n_tiles;
    return c;
}
__device__ __forceinline__ void advance(const AttnParams &p, Cursor &c) {
    if (++c.t == p.seq[c.s].n_tiles) {
        c.t = 0;
        if (++c.h == p.kv_heads) { c.h = 0; c.s++; }
    }
}
// First tile of a CTA's share.  The tile line is cut into shares of equal cost, not equal
// length: a share that begins a group pays that segment's prologue (Q load) and epilogue
// (cross-warp sum, partial write) on top of its tiles, SEG_COST tile times by measurement
// (CTAs with a group boundary inside their share finished 2.6 us after the others at
// 0.79 us per tile).  So every group is given SEG_COST virtual tiles in front of its real
// ones, the virtual line is cut evenly, and a cut that falls among the virtual tiles moves
// to the group's first real tile.
#ifndef QW_SEG_COST
#define QW_SEG_COST 3
#endif
constexpr int SEG_COST = QW_SEG_COST;
__host__ __device__ __forceinline__ int share_lo(const AttnParams &p, int cta) {
    if (cta >= p.n_cta) return p.total_tiles;
    const int64_t v_total = (int64_t)p.total_tiles + (int64_t)SEG_COST * p.n_seq * p.kv_heads;
    // (32-bit division where the product fits, which is every realistic launch: a 64-bit one is a hundred instructions
    // at the head of every CTA)
    const int64_t v = (v_total * p.n_cta) >> 31 ? ((int64_t)cta * v_total) / p.n_cta
                                                  : (int64_t)(((uint32_t)cta * (uint32_t)v_total) / (uint32_t)p.n_cta);
    int s = 0, e = p.n_seq - 1;
    while (s < e) {
        const int m = (s + e + 1) >> 1;
        if ((int64_t)p.seq[m].cum_tiles + (int64_t)SEG_COST * m * p.kv_heads <= v) s = m; else e = m - 1;
    }
    const int64_t rel = v - ((int64_t)p.seq[s].cum_tiles + (int64_t)SEG_COST * s * p.kv_heads);
    const int per = p.seq[s].n_tiles + SEG_COST;
    int h = rel >> 31 ? (int)(rel / per) : (int)((uint32_t)rel / (uint32_t)per);
    if (h > p.kv_heads - 1) h = p.kv_heads - 1;
    int o = (int)(rel - (int64_t)h * per) - SEG_COST;
    if (o < 0) o = 0;
    if (o > p.seq[s].n_tiles) o = p.seq[s].n_tiles;
    return p.seq[s].cum_tiles + h * p.seq[s].n_tiles + o;
}
// The CTAs whose shares [share_lo(c), share_lo(c + 1)) meet the tiles [G0, G1) of one group: a guess
// from the even cut, then a short walk (the cost-weighted cut moves a boundary by a few CTAs at most).
__host__ __device__ __forceinline__ void group_ctas(const AttnParams &p, int64_t G0, int64_t G1, int &c_first, int &c_last) {
    const int C = p.n_cta;
    int64_t g = (G0 * C) / p.total_tiles;
    c_first = (int)(g < C - 1 ? g : C - 1);
    while (c_first > 0 && share_lo(p, c_first) > G0) c_first--;
    while (c_first + 1 < C && share_lo(p, c_first + 1) <= G0) c_first++;
    g = ((G1 - 1) * C) / p.total_tiles;
    c_last = (int)(g < C - 1 ? g : C - 1);
    while (c_last > 0 && share_lo(p, c_last) >= G1) c_last--;
    while (c_last + 1 < C && share_lo(p, c_last + 1) < G1) c_last++;
}

__device__ __forceinline__ float load_gate(const void *g, size_t i, int dtype) {
    return dtype == DT_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(g)[i])
                            : reinterpret_cast<const float *>(g)[i];
}
__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + __expf(-x)); }
// 2^x for x <= 0 (and -inf -> 0): the hardware approximation, 2 ulp
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One CTA per SM with at most 8 warps, so every thread may use 255 registers.
template <int MT, int KG_>
__global__ void __maxnreg__((SplitCfg<MT, KG_>::MAXREG)) qw_attn_split_kernel(const __grid_constant__ AttnParams p) {
    using Cfg = SplitCfg<MT, KG_>;
    constexpr int KG = Cfg::KG, NW = Cfg::NW, NST = Cfg::NST;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *q_s = smem + Cfg::OFF_Q;
    float *red = reinterpret_cast<float *>(smem + Cfg::OFF_RED);
    float *sm_m = reinterpret_cast<float *>(smem + Cfg::OFF_M);
    float *sm_l = reinterpret_cast<float *>(smem + Cfg::OFF_L);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + Cfg::OFF_BAR);
    uint64_t *empty = full + NST;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + NST);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lo = share_lo(p, blockIdx.x), hi = share_lo(p, blockIdx.x + 1);

    if (threadIdx.x == 0) {
        for (int i = 0; i < NST; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], MT * (KG >= 2 ? 2 : 1));
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // Dependent launch.  With p.early the kernel in front is this node's own K/V append, which
    // waited for everything before it and touches only the rows [fresh_pos, ...) of each cache: what
    // this kernel reads before its wait -- cached keys, page tables, raw query rows -- was complete
    // before that kernel started, and the partial scratch is no longer in use, so only the tiles that
    // hold appended rows wait.  Otherwise the whole kernel waits here.  The kernel behind (the
    // merge) may be brought in right away: it touches nothing of ours before its own wait.
    if (!p.early) pdl_wait();
    pdl_launch_next();
    if (lo >= hi) { pdl_wait(); return; }

    if (warp == NW) {
        // ---------------- producer warp (lane 0 issues the TMA loads) ----------------
        bool waited = !p.early;
        Cursor pc = locate(p, lo);
        // the current sequence's entries of the launch table, re-read only when the cursor changes sequence
        int cur_s = -1, s_tile0 = 0, s_ntiles = 1, s_fresh = 0, s_kctx = 0, s_vctx = 0, s_kmap = 0, s_vmap = 0, s_kstride = 0, s_vstride = 0;
        const int32_t *s_ktab = nullptr, *s_vtab = nullptr;
        // page ids of 32 consecutive tiles, one per lane, fetched together: one global-memory
        // latency per 32 tiles instead of one per tile in front of every issue
        int win_k = 0, win_v = 0;
        for (int T = lo; T < hi; T++) {
            const int i = T - lo, slot = i % NST;
            if (pc.s != cur_s) {
                const AttnSeq &sq = p.seq[pc.s];
                cur_s = pc.s; s_tile0 = sq.tile0; s_ntiles = sq.n_tiles; s_fresh = sq.fresh_pos;
                s_ktab = sq.kc.table; s_vtab = sq.vc.table; s_kstride = sq.kc.pt_stride; s_vstride = sq.vc.pt_stride;
                s_kctx = sq.kc.max_ctx; s_vctx = sq.vc.max_ctx; s_kmap = sq.kmap; s_vmap = sq.vmap;
            }
            if ((i & 31) == 0) {
                const int T2 = T + lane;
                if (T2 < hi) {
                    if (pc.t + lane < s_ntiles) {                  // still in the cursor's group: no walk over the table
                        if (s_ktab) {
                            const int pg = ((s_tile0 + pc.t + lane) * TILE_KEYS) >> 6;
                            win_k = __ldg(s_ktab + (size_t)pc.h * s_kstride + pg);
                            win_v = __ldg(s_vtab + (size_t)pc.h * s_vstride + pg);
                        }
                    } else {
                        const Cursor c2 = locate(p, T2);
                        const AttnSeq &s2 = p.seq[c2.s];
                        if (s2.kc.table) {
                            const int pg = ((s2.tile0 + c2.t) * TILE_KEYS) >> 6;
                            win_k = __ldg(s2.kc.table + (size_t)c2.h * s2.kc.pt_stride + pg);
                            win_v = __ldg(s2.vc.table + (size_t)c2.h * s2.vc.pt_stride + pg);
                        }
                    }
                }
            }
            const int kp = __shfl_sync(0xffffffffu, win_k, i & 31);
            const int vp = __shfl_sync(0xffffffffu, win_v, i & 31);
            if (i >= NST) mbar_wait(&empty[slot], ((i / NST) - 1) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
            if (lane == 0) {
                const int t_abs = (s_tile0 + pc.t) * TILE_KEYS;
                // rows from fresh_pos on were appended by the kernel in front of this one
                if (!waited && t_abs + TILE_KEYS > s_fresh) { pdl_wait(); waited = true; }
                int64_t kr, vr;
                if (s_ktab) {
                    if (kp < 0 || vp < 0) report(p.status, QW_ST_BAD_PAGE);
                    kr = (int64_t)max(kp, 0) * QW_PAGE_TOKENS + (t_abs & 63);
                    vr = (int64_t)max(vp, 0) * QW_PAGE_TOKENS + (t_abs & 63);
                } else {
                    kr = (int64_t)pc.h * s_kctx + t_abs;
                    vr = (int64_t)pc.h * s_vctx + t_abs;
                }
                uint8_t *st = smem + slot * STAGE_BYTES;
                mbar_expect_tx(&full[slot], STAGE_BYTES);
#pragma unroll
                for (int b = 0; b < 4; b++) tma_load_2d(st + b * BOX_BYTES, &p.maps[s_kmap], b * 64, (int32_t)kr, &full[slot]);
#pragma unroll
                for (int b = 0; b < 4; b++)
                    tma_load_2d(st + (4 + b) * BOX_BYTES, &p.maps[s_vmap], b * 64, (int32_t)vr, &full[slot]);
            }
            if (++pc.t == s_ntiles) {                              // (advance(), on the cached tile count)
                pc.t = 0;
                if (++pc.h == p.kv_heads) { pc.h = 0; pc.s++; }
            }
            __syncwarp();
        }
        // falls through to the end: consumers wait for every stage that was issued.
        if (lane == 0 && !waited) pdl_wait();      // every CTA has waited before it exits
    } else {
        // ---------------- consumers ----------------
        const int mt = warp / KG, kg = warp % KG;
        const int gid = lane >> 2, tig = lane & 3;
        const uint32_t q_base = smem_u32(q_s);
        const float sc2 = p.scale * LOG2E;

        float o[32][4];
        float m0, m1, l0, l1;
        Cursor c = locate(p, lo);
        int T = lo;
        while (T < hi) {
            // ---- segment start ----
            const AttnSeq &sq = p.seq[c.s];
            const int seg_t0 = c.t;
            const int seg_n = min(sq.n_tiles - c.t, hi - T);
            const int valid_rows = sq.rows * p.gqa;
            const int head0 = c.h * p.gqa;

            // Q of this group -> bf16, swizzled: 4 boxes of [MT*16 rows, 64 dims].
            if (p.q_raw) {
                // Raw rows of the [q|gate] projection: per-head RMS norm and partial RoPE here, in the
                // arithmetic of the pre-op kernel (qwasar_cpu.c:68-82, 304-319), one warp per row, lane l
                // holding dims 8l .. 8l+7.  The rows' cos / sin (one angle per lane) go through the
                // reduction buffer, which is idle until the segment ends.  The first rows are requested
                // before the angles are worked out, so the two trips to memory overlap.
                constexpr int PF = 4;                              // rows a warp has in flight
                float *cs = red;
                uint4 raw[PF][2];
                auto fetch = [&](int row, uint4 (&r2)[2]) {
                    r2[0] = make_uint4(0, 0, 0, 0); r2[1] = r2[0];
                    if (row >= valid_rows) return;
                    const int r = row / p.gqa, g = row - r * p.gqa;
                    const size_t src = ((size_t)r * p.q_heads + head0 + g) * 512 + lane * 8;
                    if (p.q_dtype == DT_BF16) {
                        r2[0] = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(sq.q) + src));
                    } else {
                        const uint4 *g4 = reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(sq.q) + src);
                        r2[0] = __ldg(g4); r2[1] = __ldg(g4 + 1);
                    }
                };
#pragma unroll
                for (int u = 0; u < PF; u++) fetch(warp + u * NW, raw[u]);
                uint4 w4 = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
                if (p.q_norm_w) w4 = __ldg(reinterpret_cast<const uint4 *>(p.q_norm_w) + lane);
                {
                    // the token's position on all three axes and the dim's axis side by side (a position
                    // looked up through the axis would be a second trip to memory)
                    const int ax = p.axis[lane];
                    const float fr = p.inv_freq[lane];
                    for (int r = warp; r < sq.rows; r += NW) {
                        const int32_t p0 = sq.pos[r], p1 = sq.pos[(size_t)sq.pos_stride + r], p2 = sq.pos[(size_t)2 * sq.pos_stride + r];
                        const float ang = __fmul_rn((float)(ax == 0 ? p0 : ax == 1 ? p1 : p2), fr);
                        // cos / sin of the fp32 angle (it reaches 2^18 rad): the remainder modulo 2 pi in
                        // double precision, good to 1e-10, then the fast functions on [-pi, pi] (2^-21) --
                        // far below the bf16 rounding the query gets next
                        const double turns = rint((double)ang * 0.15915494309189535);
                        const float rem = (float)fma(turns, -6.283185307179586, (double)ang);
                        float sn, cn;
                        __sincosf(rem, &sn, &cn);
                        cs[r * 64 + lane] = cn; cs[r * 64 + 32 + lane] = sn;
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
                const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
                auto finish = [&](int row, const uint4 (&r2)[2]) {
                    uint4 val = make_uint4(0, 0, 0, 0);
                    if (row < valid_rows) {
                        const int r = row / p.gqa;
                        float x[8];
                        if (p.q_dtype == DT_BF16) {
                            const uint32_t xw[4] = {r2[0].x, r2[0].y, r2[0].z, r2[0].w};
#pragma unroll
                            for (int i = 0; i < 4; i++) { x[2 * i] = __uint_as_float(xw[i] << 16); x[2 * i + 1] = __uint_as_float(xw[i] & 0xffff0000u); }
                        } else {
                            x[0] = __uint_as_float(r2[0].x); x[1] = __uint_as_float(r2[0].y); x[2] = __uint_as_float(r2[0].z); x[3] = __uint_as_float(r2[0].w);
                            x[4] = __uint_as_float(r2[1].x); x[5] = __uint_as_float(r2[1].y); x[6] = __uint_as_float(r2[1].z); x[7] = __uint_as_float(r2[1].w);
                        }
                        float ss = 0.0f;
#pragma unroll
                        for (int i = 0; i < 8; i++) ss = __fadd_rn(ss, __fmul_rn(x[i], x[i]));
                        ss = warp_sum(ss);
                        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 256.0f), p.eps)));
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            x[i] = __fmul_rn(x[i], inv);
                            if (p.q_norm_w) x[i] = __fmul_rn(x[i], __uint_as_float((i & 1) ? (ww[i >> 1] & 0xffff0000u) : (ww[i >> 1] << 16)));
                        }
                        // dims d < 32 sit in lanes 0-3, their partners d + 32 in lanes 4-7
                        const float *cr = cs + r * 64 + 8 * (lane & 3);
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const float other = __shfl_xor_sync(0xffffffffu, x[i], 4);
                            if (lane < 8) {
                                const float cn = cr[i], sn = cr[32 + i];
                                x[i] = lane < 4 ? __fsub_rn(__fmul_rn(x[i], cn), __fmul_rn(other, sn))
                                                : __fadd_rn(__fmul_rn(x[i], cn), __fmul_rn(other, sn));
                            }
                        }
                        val = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
                    }
                    *reinterpret_cast<uint4 *>(q_s + (lane >> 3) * (MT * 16 * 128) + swz128(row, (lane & 7) * 8)) = val;
                };
                for (int row0 = warp; row0 < MT * 16; row0 += NW * PF) {
                    if (row0 != warp) {
#pragma unroll
                        for (int u = 0; u < PF; u++) fetch(row0 + u * NW, raw[u]);
                    }
#pragma unroll
                    for (int u = 0; u < PF; u++)
                        if (row0 + u * NW < MT * 16) finish(row0 + u * NW, raw[u]);
                }
            } else
            for (int idx = warp * 32 + lane; idx < MT * 16 * 32; idx += NW * 32) {
                const int row = idx >> 5, chunk = idx & 31;           // 16-byte chunk = 8 dims
                uint4 val = make_uint4(0, 0, 0, 0);
                if (row < valid_rows) {
                    const int r = row / p.gqa, g = row - r * p.gqa;
                    const size_t src = ((size_t)r * p.q_heads + head0 + g) * 256 + chunk * 8;
                    if (p.q_dtype == DT_BF16) {
                        val = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(sq.q) + src);
                    } else {
                        const float4 a = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(sq.q) + src);
                        const float4 b = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(sq.q) + src + 4);
                        val.x = pack_bf16(a.x, a.y); val.y = pack_bf16(a.z, a.w);
                        val.z = pack_bf16(b.x, b.y); val.w = pack_bf16(b.z, b.w);
                    }
                }
                *reinterpret_cast<uint4 *>(q_s + (chunk >> 3) * (MT * 16 * 128) + swz128(row, (chunk & 7) * 8)) = val;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");

#pragma unroll
            for (int n = 0; n < 32; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
            m0 = m1 = NEG_BIG;
            l0 = l1 = 0.0f;

            // causal limits of this thread's two rows (last readable key index)
            const int row0 = mt * 16 + gid, row1 = row0 + 8;
            // The segment's constants are pinned in registers: read through `sq` inside the tile loop they are
            // indexed loads from the launch's sequence table, which stops fitting the constant cache beyond a
            // dozen sequences (the kernel lost 12 % at 32 sequences and 22 % at 64 before this).
            int key_hi = sq.key_hi, seg_tile0 = sq.tile0 + seg_t0;
            asm volatile("" : "+r"(key_hi), "+r"(seg_tile0));
            const int lim0 = min(key_hi - 1, row0 < valid_rows ? sq.base_pos + row0 / p.gqa : 0x7fffffff);
            const int lim1 = min(key_hi - 1, row1 < valid_rows ? sq.base_pos + row1 / p.gqa : 0x7fffffff);
            const int mask_from = min(key_hi, sq.base_pos + 1);   // blocks reaching this key need masking

            for (int tt = 0; tt < seg_n; tt++, T++) {
                const int i = T - lo, slot = i % NST;
                bool uses = false;
#pragma unroll
                for (int j = 0; j < 2; j++) uses |= ((2 * i + j) % KG) == kg;
                if (!uses) continue;
                mbar_wait(&full[slot], (i / NST) & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                const uint32_t k_base = smem_u32(smem + slot * STAGE_BYTES);
                const uint32_t v_base = k_base + 4 * BOX_BYTES;
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    if (((2 * i + j) % KG) != kg) continue;
                    const int blk_t0 = (seg_tile0 + tt) * TILE_KEYS + j * 16;
                    if (blk_t0 >= key_hi) continue;

                    // ---- S = Q K^T for 16 keys ----
                    // fragments of k-step ks+1 are requested before the tensor ops of step ks
                    // are issued, so shared-memory latency hides behind them; two accumulator
                    // sets halve the dependent chain
                    float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
                    float s2[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
                    {
                        const int mi = lane >> 3;
                        const uint32_t q_row = mt * 16 + (mi & 1) * 8 + (lane & 7);
                        const uint32_t k_row = j * 16 + (mi >> 1) * 8 + (lane & 7);
                        uint32_t qa[2][4], kb[2][4];
                        auto fetch = [&](int ks, uint32_t(&a)[4], uint32_t(&b)[4]) {
                            const uint32_t qc = ks * 2 + (mi >> 1), kc = ks * 2 + (mi & 1);
                            ldsm_x4(a[0], a[1], a[2], a[3], q_base + (qc >> 3) * (MT * 16 * 128) + swz128(q_row, (qc & 7) * 8));
                            ldsm_x4(b[0], b[1], b[2], b[3], k_base + (kc >> 3) * BOX_BYTES + swz128(k_row, (kc & 7) * 8));
                        };
                        fetch(0, qa[0], kb[0]);
#pragma unroll
                        for (int ks = 0; ks < 16; ks++) {
                            if (ks + 1 < 16) fetch(ks + 1, qa[(ks + 1) & 1], kb[(ks + 1) & 1]);
                            const uint32_t(&a)[4] = qa[ks & 1];
                            const uint32_t(&b)[4] = kb[ks & 1];
                            if (ks & 1) {
                                mma_bf16(s2[0], a[0], a[1], a[2], a[3], b[0], b[1]);
                                mma_bf16(s2[1], a[0], a[1], a[2], a[3], b[2], b[3]);
                            } else {
                                mma_bf16(s[0], a[0], a[1], a[2], a[3], b[0], b[1]);
                                mma_bf16(s[1], a[0], a[1], a[2], a[3], b[2], b[3]);
                            }
                        }
                    }
#pragma unroll
                    for (int n = 0; n < 2; n++)
#pragma unroll
                        for (int e = 0; e < 4; e++) s[n][e] = (s[n][e] + s2[n][e]) * sc2;

                    if (blk_t0 + 16 > mask_from) {
#pragma unroll
                        for (int n = 0; n < 2; n++)
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const int key = blk_t0 + n * 8 + tig * 2 + (e & 1);
                                if (key > ((e & 2) ? lim1 : lim0)) s[n][e] = -INFINITY;
                            }
                    }

                    // ---- online softmax ----
                    float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
                    float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
                    if (__any_sync(0xffffffffu, (mn0 > m0) || (mn1 > m1))) {
                        const float al0 = ex2(m0 - mn0), al1 = ex2(m1 - mn1);
                        l0 *= al0; l1 *= al1;
#pragma unroll
                        for (int n = 0; n < 32; n++) { o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1; }
                        m0 = mn0; m1 = mn1;
                    }
                    uint32_t pa[4];
                    {
                        const float p00 = ex2(s[0][0] - m0), p01 = ex2(s[0][1] - m0);
                        const float p02 = ex2(s[0][2] - m1), p03 = ex2(s[0][3] - m1);
                        const float p10 = ex2(s[1][0] - m0), p11 = ex2(s[1][1] - m0);
                        const float p12 = ex2(s[1][2] - m1), p13 = ex2(s[1][3] - m1);
                        l0 += (p00 + p01) + (p10 + p11);
                        l1 += (p02 + p03) + (p12 + p13);
                        pa[0] = pack_bf16(p00, p01); pa[1] = pack_bf16(p02, p03);
                        pa[2] = pack_bf16(p10, p11); pa[3] = pack_bf16(p12, p13);
                    }

                    // ---- O += P V ----
                    {
                        const int mi = lane >> 3;
                        const uint32_t v_row = j * 16 + (mi & 1) * 8 + (lane & 7);
                        const bool ragged = blk_t0 + 16 > key_hi;   // keys past the end may hold anything
                        const int k_a = blk_t0 + tig * 2;              // key of a b-register's low half (b0); +8 for b1
                        const uint32_t keep_a = (k_a < key_hi ? 0x0000ffffu : 0u) | (k_a + 1 < key_hi ? 0xffff0000u : 0u);
                        const uint32_t keep_b = (k_a + 8 < key_hi ? 0x0000ffffu : 0u) | (k_a + 9 < key_hi ? 0xffff0000u : 0u);
                        uint32_t vb[2][4];
                        auto fetch_v = [&](int np, uint32_t(&b)[4]) {
                            const uint32_t vc = np * 2 + (mi >> 1);
                            ldsm_x4_t(b[0], b[1], b[2], b[3], v_base + (vc >> 3) * BOX_BYTES + swz128(v_row, (vc & 7) * 8));
                        };
                        fetch_v(0, vb[0]);
#pragma unroll
                        for (int np = 0; np < 16; np++) {
                            if (np + 1 < 16) fetch_v(np + 1, vb[(np + 1) & 1]);
                            uint32_t b0 = vb[np & 1][0], b1 = vb[np & 1][1], b2 = vb[np & 1][2], b3 = vb[np & 1][3];
                            if (ragged) { b0 &= keep_a; b2 &= keep_a; b1 &= keep_b; b3 &= keep_b; }
                            mma_bf16(o[np * 2], pa[0], pa[1], pa[2], pa[3], b0, b1);
                            mma_bf16(o[np * 2 + 1], pa[0], pa[1], pa[2], pa[3], b2, b3);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);
            }

            // ---- segment end: merge the KG warps of each row tile ----
            l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
            if (tig == 0) {
                sm_m[(mt * KG + kg) * 16 + gid] = m0;
                sm_m[(mt * KG + kg) * 16 + gid + 8] = m1;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
            float M0 = NEG_BIG, M1 = NEG_BIG;
#pragma unroll
            for (int g2 = 0; g2 < KG; g2++) {
                M0 = fmaxf(M0, sm_m[(mt * KG + g2) * 16 + gid]);
                M1 = fmaxf(M1, sm_m[(mt * KG + g2) * 16 + gid + 8]);
            }
            {
                // the KG warps of a row tile add their accumulators into `red` one after the
                // other (plain loads and stores, valid rows only): KG short rounds instead of
                // thousands of conflicting shared-memory atomics
                const float f0 = ex2(m0 - M0), f1 = ex2(m1 - M1);
                const bool v0 = mt * 16 + gid < valid_rows, v1 = mt * 16 + gid + 8 < valid_rows;
                float2 *r0 = reinterpret_cast<float2 *>(red + (size_t)(mt * 16 + gid) * RED_LD + tig * 2);
                float2 *r1 = r0 + 8 * (RED_LD / 2);
                const bool two_chains = MT == 1 && KG >= 2 && valid_rows <= 8;
                if (two_chains) {
                    // At most 8 valid rows (a decode step): rows 8-15 of `red` are free, so the odd key groups add
                    // up there while the even ones use rows 0-7 -- half the rounds; the reader adds the two halves.
                    float2 *rr = (kg & 1) ? r1 : r0;
                    const int lrow = mt * 16 + gid + ((kg & 1) ? 8 : 0);
#pragma unroll 1
                    for (int round = 0; round < (KG + 1) / 2; round++) {
                        if ((kg >> 1) == round) {
                            if (v0) {
                                if (round == 0) {
#pragma unroll
                                    for (int n = 0; n < 32; n++) rr[n * 4] = make_float2(o[n][0] * f0, o[n][1] * f0);
                                } else {
#pragma unroll
                                    for (int n = 0; n < 32; n++) {
                                        const float2 t = rr[n * 4];
                                        rr[n * 4] = make_float2(fmaf(o[n][0], f0, t.x), fmaf(o[n][1], f0, t.y));
                                    }
                                }
                            }
                            if (tig == 0) sm_l[lrow] = (round ? sm_l[lrow] : 0.0f) + l0 * f0;
                        }
                        asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
                    }
                } else
#pragma unroll 1
                for (int round = 0; round < KG; round++) {
                    if (kg == round) {
                        if (round == 0) {
                            if (v0) {
#pragma unroll
                                for (int n = 0; n < 32; n++) r0[n * 4] = make_float2(o[n][0] * f0, o[n][1] * f0);
                            }
                            if (v1) {
#pragma unroll
                                for (int n = 0; n < 32; n++) r1[n * 4] = make_float2(o[n][2] * f1, o[n][3] * f1);
                            }
                            if (tig == 0) { sm_l[mt * 16 + gid] = l0 * f0; sm_l[mt * 16 + gid + 8] = l1 * f1; }
                        } else {
                            if (v0) {
#pragma unroll
                                for (int n = 0; n < 32; n++) {
                                    float2 t = r0[n * 4];
                                    r0[n * 4] = make_float2(fmaf(o[n][0], f0, t.x), fmaf(o[n][1], f0, t.y));
                                }
                            }
                            if (v1) {
#pragma unroll
                                for (int n = 0; n < 32; n++) {
                                    float2 t = r1[n * 4];
                                    r1[n * 4] = make_float2(fmaf(o[n][2], f1, t.x), fmaf(o[n][3], f1, t.y));
                                }
                            }
                            if (tig == 0) { sm_l[mt * 16 + gid] += l0 * f0; sm_l[mt * 16 + gid + 8] += l1 * f1; }
                        }
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
                }
            }

            const bool whole = (seg_t0 == 0) && (seg_n == sq.n_tiles) && (p.mode == 0);
            const int slot_id = blockIdx.x + c.s * p.kv_heads + c.h;   // partial slot of (cta, group)
            for (int idx = warp * 32 + lane; idx < valid_rows * 64; idx += NW * 32) {
                const int row = idx >> 6, d4 = (idx & 63) * 4;
                float4 acc = *reinterpret_cast<const float4 *>(red + (size_t)row * RED_LD + d4);
                float Mrow = NEG_BIG;
#pragma unroll
                for (int g2 = 0; g2 < KG; g2++) Mrow = fmaxf(Mrow, sm_m[((row >> 4) * KG + g2) * 16 + (row & 15)]);
                float L = sm_l[row];
                if (MT == 1 && KG >= 2 && valid_rows <= 8) {       // (the odd key groups' half, see above)
                    const float4 hi = *reinterpret_cast<const float4 *>(red + (size_t)(row + 8) * RED_LD + d4);
                    acc.x += hi.x; acc.y += hi.y; acc.z += hi.z; acc.w += hi.w;
                    L += sm_l[row + 8];
                }
                if (whole) {
                    const int r = row / p.gqa, g = row - r * p.gqa;
                    const size_t oi = ((size_t)r * p.q_heads + head0 + g) * 256 + d4;
                    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
                    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
                    if (sq.gate) {
                        const size_t gi = ((size_t)r * p.q_heads + head0 + g) * p.gate_stride + d4;
                        acc.x *= sigmoidf(load_gate(sq.gate, gi, p.gate_dtype));
                        acc.y *= sigmoidf(load_gate(sq.gate, gi + 1, p.gate_dtype));
                        acc.z *= sigmoidf(load_gate(sq.gate, gi + 2, p.gate_dtype));
                        acc.w *= sigmoidf(load_gate(sq.gate, gi + 3, p.gate_dtype));
                    }
                    if (p.out_dtype == DT_BF16) {
                        uint2 v;
                        v.x = pack_bf16(acc.x, acc.y); v.y = pack_bf16(acc.z, acc.w);
                        *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(sq.out) + oi) = v;
                    } else {
                        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(sq.out) + oi) = acc;
                    }
                } else {
                    const size_t pi = (size_t)slot_id * (MT * 16) + row;
                    *reinterpret_cast<float4 *>(p.pacc + pi * 256 + d4) = acc;
                    if ((idx & 63) == 0) {
                        p.pstat[pi * 2] = Mrow * LN2;
                        p.pstat[pi * 2 + 1] = L;
                    }
                }
            }
            // next segment (if any) begins with the next group
            for (int k2 = 0; k2 < seg_n; k2++) advance(p, c);
            asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
        }
    }
}

// ---- the exchange of partials between GPUs (a sequence split by position) ----------------
// A record is one (row, head)'s combined partial: acc[256], max (natural units), sum, padded to
// XCHG_REC floats so that records stay 16-byte aligned.  Rank a's record of epoch e goes to slot
// [e & 1][a][rh] of EVERY rank's gather buffer by plain stores (peer stores over NVLink for the
// others), then, after a system-wide fence, the epoch number goes into the flag beside it.  A rank
// merges when the flags of all ranks show the epoch.  Two parities suffice: a rank can only publish
// epoch e + 2 after it has merged epoch e + 1, which needed every rank's record of e + 1, which
// those ranks published after they had merged epoch e.
constexpr int XCHG_REC = QW_XCHG_REC;

__device__ __forceinline__ void st_release_sys(int *p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int *p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Threads 0-63 of a block, each holding four dims (d4 ..) of the combined partial of (row, head) rh.
__device__ __forceinline__ void xchg_publish(const XchgDev &x, size_t ci, int tid, int d4, float4 acc, float m, float den) {
    const size_t slot = (size_t)((x.epoch & 1) * x.n_ranks + x.rank) * x.max_rh + ci;
    for (int i = 0; i < x.n_ranks; i++) {
        float *rec = x.gather[i] + slot * XCHG_REC;
        *reinterpret_cast<float4 *>(rec + d4) = acc;
        if (tid == 0) { rec[256] = den > 0.0f ? m : -3.0e38f; rec[257] = den; }
    }
    __threadfence_system();
    asm volatile("bar.sync 1, 64;" ::: "memory");
    if (tid < x.n_ranks) st_release_sys(x.flags[tid] + slot, x.epoch);
}

// Waits (bounded) for every rank's record of this epoch, merges them by log-sum-exp, applies the
// gate and writes the output row.  Threads 0-63 of a block.
__device__ __forceinline__ void xchg_collect(const AttnParams &p, const AttnSeq &sq, size_t ci, size_t rh, int tid, int d4, int *late_s) {
    const XchgDev &x = p.x;
    const size_t slot0 = (size_t)((x.epoch & 1) * x.n_ranks) * x.max_rh + ci;
    float gate4[4] = {0.f, 0.f, 0.f, 0.f};
    if (sq.gate) {
        const size_t gi = rh * p.gate_stride + d4;
#pragma unroll
        for (int i = 0; i < 4; i++) gate4[i] = load_gate(sq.gate, gi + i, p.gate_dtype);
    }
    if (tid < x.n_ranks) {
        const int *f = x.flags[x.rank] + slot0 + (size_t)tid * x.max_rh;
        const uint64_t t0 = global_ns();
        while (ld_acquire_sys(f) != x.epoch) {
            if ((int64_t)(global_ns() - t0) > x.timeout_ns) { *late_s = 1; break; }
            __nanosleep(100);
        }
    }
    asm volatile("bar.sync 1, 64;" ::: "memory");
    if (*reinterpret_cast<volatile int *>(late_s)) {
        if (tid == 0) report(p.status, QW_ST_PEER_TIMEOUT);
        return;
    }
    const float *mine = x.gather[x.rank] + slot0 * XCHG_REC;
    float m = -3.0e38f;
    for (int i = 0; i < x.n_ranks; i++) {
        const float2 st = __ldcg(reinterpret_cast<const float2 *>(mine + (size_t)i * x.max_rh * XCHG_REC + 256));
        if (st.y > 0.0f) m = fmaxf(m, st.x);
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.0f;
    for (int i = 0; i < x.n_ranks; i++) {
        const float *rec = mine + (size_t)i * x.max_rh * XCHG_REC;
        const float2 st = __ldcg(reinterpret_cast<const float2 *>(rec + 256));
        const float w = st.y > 0.0f ? __expf(st.x - m) : 0.0f;
        const float4 a = __ldcg(reinterpret_cast<const float4 *>(rec + d4));
        den += st.y * w;
        acc.x += a.x * w; acc.y += a.y * w; acc.z += a.z * w; acc.w += a.w * w;
    }
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    if (sq.gate) {
        acc.x *= sigmoidf(gate4[0]); acc.y *= sigmoidf(gate4[1]); acc.z *= sigmoidf(gate4[2]); acc.w *= sigmoidf(gate4[3]);
    }
    if (p.out_dtype == DT_BF16) {
        uint2 v;
        v.x = pack_bf16(acc.x, acc.y); v.y = pack_bf16(acc.z, acc.w);
        *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(sq.out) + rh * 256 + d4) = v;
    } else {
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(sq.out) + rh * 256 + d4) = acc;
    }
}

// One block per (group, row i): combine the group's partials.  A group cut over many CTAs (one
// long sequence: up to one partial per SM) must not be walked one partial at a time -- every
// step of such a walk is a trip to L2 -- so the block reads all (max, sum) pairs at once, one per
// thread, and its four quarters of 64 threads x float4 each take every fourth partial, four
// loads in flight, before their sums are added through shared memory.
constexpr int MERGE_THREADS = 256;
template <int MT>
__global__ void __launch_bounds__(MERGE_THREADS) qw_attn_merge_kernel(const __grid_constant__ AttnParams p, int max_valid_rows) {
    __shared__ float w_s[MERGE_THREADS];                      // weight of partial q (0 for an empty one)
    __shared__ float red_s[2][8];
    __shared__ __align__(16) float acc_s[3][256];
    __shared__ int late_s;
    // Dependent launch: the kernel behind this one touches nothing before its own wait, so it may
    // be brought in at once; this kernel reads partials, and writes, only after its wait.  Every
    // block waits before it exits.
    pdl_launch_next();
    const int gidx = blockIdx.x / max_valid_rows;            // sequence * kv_heads + head
    const int row = blockIdx.x - gidx * max_valid_rows;
    const int s = gidx / p.kv_heads, h = gidx - s * p.kv_heads;
    if (s >= p.n_seq) { pdl_wait(); return; }
    const AttnSeq &sq = p.seq[s];
    if (row >= sq.rows * p.gqa) { pdl_wait(); return; }
    const int64_t G0 = (int64_t)sq.cum_tiles + (int64_t)h * sq.n_tiles, G1 = G0 + sq.n_tiles;
    int c_first, c_last;
    group_ctas(p, G0, G1, c_first, c_last);
    const int parts = c_last - c_first + 1;                   // <= n_cta <= MERGE_THREADS
    if (parts == 1 && p.mode == 0) { pdl_wait(); return; }    // the split kernel wrote the output itself

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const size_t pi0 = (size_t)(c_first + gidx) * (MT * 16) + row;      // partial q sits MT*16 rows further per q
    // the gate of the row is fetched now, by the quarter that will use it: it depends on nothing here
    const int r = row / p.gqa, g = row - r * p.gqa;
    const size_t rh = (size_t)r * p.q_heads + h * p.gqa + g;
    if (tid == 0) late_s = 0;
    if (p.mode == 4 || (p.mode >= 2 && p.x.empty)) {
        // the second half of an exchange alone (the records are already on their way), or a rank
        // whose range holds no visible key: it publishes an empty record (sum 0 drops out of the merge)
        pdl_wait();
        if (tid >= 64) return;
        asm volatile("bar.sync 1, 64;" ::: "memory");
        const size_t ci = (size_t)sq.row_slot0 * p.q_heads + rh;
        if (p.mode != 4) xchg_publish(p.x, ci, tid, tid * 4, make_float4(0.f, 0.f, 0.f, 0.f), -3.0e38f, 0.0f);
        if (p.mode != 3) xchg_collect(p, sq, ci, rh, tid, tid * 4, &late_s);
        return;
    }
    float gate4[4] = {0.f, 0.f, 0.f, 0.f};
    if (sq.gate && p.mode == 0 && tid < 64) {
        const size_t gi = rh * p.gate_stride + tid * 4;
#pragma unroll
        for (int i = 0; i < 4; i++) gate4[i] = load_gate(sq.gate, gi + i, p.gate_dtype);
    }
    pdl_wait();
    // the first accumulators of this thread's quarter are asked for together with the (max, sum) pairs: their
    // weights are not needed until they arrive, and one trip to L2 is saved
    const int quarter = tid >> 6, d4 = (tid & 63) * 4;
    const float *base = p.pacc + pi0 * 256 + d4;
    const size_t step = (size_t)(MT * 16) * 256;
    float4 first[4];
#pragma unroll
    for (int u = 0; u < 4; u++)
        first[u] = quarter + 4 * u < parts ? *reinterpret_cast<const float4 *>(base + (size_t)(quarter + 4 * u) * step) : make_float4(0.f, 0.f, 0.f, 0.f);
    // max over the non-empty partials, then each partial's weight and the denominator
    float mq = -3.0e38f, lq = 0.0f;
    if (tid < parts) {
        const float2 st = *reinterpret_cast<const float2 *>(p.pstat + (pi0 + (size_t)tid * (MT * 16)) * 2);
        lq = st.y;
        if (lq > 0.0f) mq = st.x;
    }
    float m = warp_max(mq);
    if (lane == 0) red_s[0][warp] = m;
    __syncthreads();
    m = red_s[0][0];
#pragma unroll
    for (int i = 1; i < MERGE_THREADS / 32; i++) m = fmaxf(m, red_s[0][i]);
    const float wq = lq > 0.0f ? __expf(mq - m) : 0.0f;
    w_s[tid] = wq;
    float den = warp_sum(lq * wq);
    if (lane == 0) red_s[1][warp] = den;
    __syncthreads();
    den = 0.0f;
#pragma unroll
    for (int i = 0; i < MERGE_THREADS / 32; i++) den += red_s[1][i];

    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const float w = quarter + 4 * u < parts ? w_s[quarter + 4 * u] : 0.0f;
        acc.x += first[u].x * w; acc.y += first[u].y * w; acc.z += first[u].z * w; acc.w += first[u].w * w;
    }
    int q = quarter + 16;
    for (; q + 12 < parts; q += 16) {
        float4 a[4];
#pragma unroll
        for (int u = 0; u < 4; u++) a[u] = *reinterpret_cast<const float4 *>(base + (size_t)(q + 4 * u) * step);
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const float w = w_s[q + 4 * u];
            acc.x += a[u].x * w; acc.y += a[u].y * w; acc.z += a[u].z * w; acc.w += a[u].w * w;
        }
    }
    for (; q < parts; q += 4) {
        const float4 a = *reinterpret_cast<const float4 *>(base + (size_t)q * step);
        const float w = w_s[q];
        acc.x += a.x * w; acc.y += a.y * w; acc.z += a.z * w; acc.w += a.w * w;
    }
    if (quarter > 0) *reinterpret_cast<float4 *>(&acc_s[quarter - 1][d4]) = acc;
    __syncthreads();
    if (quarter > 0) return;
#pragma unroll
    for (int i = 0; i < 3; i++) {
        const float4 o = *reinterpret_cast<const float4 *>(&acc_s[i][d4]);
        acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
    }
    if (p.mode == 1) {
        // leave one combined partial per (row, head) for the exchange between GPUs
        const size_t ci = (size_t)sq.row_slot0 * p.q_heads + rh;
        float *ca = p.comb_acc, *cs = p.comb_stat;
        *reinterpret_cast<float4 *>(ca + ci * 256 + d4) = acc;
        if (threadIdx.x == 0) { cs[ci * 2] = den > 0.0f ? m : -3.0e38f; cs[ci * 2 + 1] = den; }
        return;
    }
    if (p.mode >= 2) {
        const size_t ci = (size_t)sq.row_slot0 * p.q_heads + rh;
        xchg_publish(p.x, ci, tid, d4, acc, m, den);
        if (p.mode == 2) xchg_collect(p, sq, ci, rh, tid, d4, &late_s);
        return;
    }
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    if (sq.gate) {
        acc.x *= sigmoidf(gate4[0]); acc.y *= sigmoidf(gate4[1]); acc.z *= sigmoidf(gate4[2]); acc.w *= sigmoidf(gate4[3]);
    }
    if (p.out_dtype == DT_BF16) {
        uint2 v;
        v.x = pack_bf16(acc.x, acc.y); v.y = pack_bf16(acc.z, acc.w);
        *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(sq.out) + rh * 256 + d4) = v;
    } else {
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(sq.out) + rh * 256 + d4) = acc;
    }
}

// ---- merge of partials laid out by part ------------------------------------------------------
// pacc [parts, n_rh, 256], pstat [parts, n_rh, 2] (max in natural units, sum): partials gathered
// from other GPUs, the slices of the per-query kernel, the chunks of the masked kernel.  One block
// per (row, head); like qw_attn_merge_kernel it reads every (max, sum) pair at once -- one per
// thread, in rounds of 256 -- and its four quarters of 64 threads x float4 each take every fourth
// part with four loads in flight, because a walk through the parts is a trip to L2 per step.  A part
// with sum 0 is not read at all (its accumulator may hold anything).
__global__ void __launch_bounds__(256) merge_parts_kernel(void *out, int out_dtype, const float *__restrict__ pacc,
                                                          const float *__restrict__ pstat, const void *gate,
                                                          int gate_dtype, int gate_stride, int n_rh, int parts,
                                                          float *pacc_out, float *pstat_out, size_t acc_stride,
                                                          size_t stat_stride) {
    __shared__ float red_s[2][8];
    __shared__ __align__(16) float acc_s[3][256];
    extern __shared__ float w_dyn[];                          // parts weights
    const int rh = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_launch_next();
    pdl_wait();
    float mq = -3.0e38f;
    for (int q = tid; q < parts; q += 256) {
        const float2 st = *reinterpret_cast<const float2 *>(pstat + (size_t)q * stat_stride + (size_t)rh * 2);
        w_dyn[q] = st.y > 0.0f ? st.x : -3.0e38f;             // the part's max for now
        if (st.y > 0.0f) mq = fmaxf(mq, st.x);
    }
    float m = warp_max(mq);
    if (lane == 0) red_s[0][warp] = m;
    __syncthreads();
    m = red_s[0][0];
#pragma unroll
    for (int i = 1; i < 8; i++) m = fmaxf(m, red_s[0][i]);
    float den = 0.0f;
    for (int q = tid; q < parts; q += 256) {
        const float l = pstat[(size_t)q * stat_stride + (size_t)rh * 2 + 1];
        const float w = l > 0.0f ? __expf(w_dyn[q] - m) : 0.0f;
        w_dyn[q] = w;
        den += l * w;
    }
    den = warp_sum(den);
    if (lane == 0) red_s[1][warp] = den;
    __syncthreads();
    den = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) den += red_s[1][i];

    const int quarter = tid >> 6, d4 = (tid & 63) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float *base = pacc + (size_t)rh * 256 + d4;
    int q = quarter;
    for (; q + 12 < parts; q += 16) {
        float4 a[4];
        float w[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            w[u] = w_dyn[q + 4 * u];
            a[u] = w[u] > 0.0f ? *reinterpret_cast<const float4 *>(base + (size_t)(q + 4 * u) * acc_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) { acc.x += a[u].x * w[u]; acc.y += a[u].y * w[u]; acc.z += a[u].z * w[u]; acc.w += a[u].w * w[u]; }
    }
    for (; q < parts; q += 4) {
        const float w = w_dyn[q];
        if (w > 0.0f) {
            const float4 a = *reinterpret_cast<const float4 *>(base + (size_t)q * acc_stride);
            acc.x += a.x * w; acc.y += a.y * w; acc.z += a.z * w; acc.w += a.w * w;
        }
    }
    if (quarter > 0) *reinterpret_cast<float4 *>(&acc_s[quarter - 1][d4]) = acc;
    __syncthreads();
    if (quarter > 0) return;
#pragma unroll
    for (int i = 0; i < 3; i++) {
        const float4 o = *reinterpret_cast<const float4 *>(&acc_s[i][d4]);
        acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
    }
    if (pacc_out) {
        *reinterpret_cast<float4 *>(pacc_out + (size_t)rh * 256 + d4) = acc;
        if (tid == 0) { pstat_out[rh * 2] = den > 0.0f ? m : -3.0e38f; pstat_out[rh * 2 + 1] = den; }
        return;
    }
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    if (gate) {
        const size_t gi = (size_t)rh * gate_stride + d4;
        acc.x *= sigmoidf(load_gate(gate, gi, gate_dtype));
        acc.y *= sigmoidf(load_gate(gate, gi + 1, gate_dtype));
        acc.z *= sigmoidf(load_gate(gate, gi + 2, gate_dtype));
        acc.w *= sigmoidf(load_gate(gate, gi + 3, gate_dtype));
    }
    if (out_dtype == DT_BF16) {
        uint2 v;
        v.x = pack_bf16(acc.x, acc.y); v.y = pack_bf16(acc.z, acc.w);
        *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(out) + (size_t)rh * 256 + d4) = v;
    } else {
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + (size_t)rh * 256 + d4) = acc;
    }
}

// ---- masked attention on tensor ops: the listed positions, gathered -----------------------------
// What qw_op_attn_masked runs when a selection exists (qwasar_gpu.h:635-651; the reference's tensor
// form is metal4/attn_tensor.metal:482-591): row r attends only the positions of its list.  The
// list's capacity is cut into chunks of 64 entries; one CTA of four warps per (chunk, kv head, row),
// a warp per 16 listed keys.  The keys' K and V rows are gathered from wherever they lie (plain
// cache or paged arena) by 16-byte asynchronous copies -- all 32 rows of a warp in flight at once,
// entries past the count or outside the cache arrive as zeros -- into the swizzled layout the
// ldmatrix fragments expect; S = Q K^T and O = P V are m16n8k16 bf16 tensor ops for all query heads
// of the kv head (rows 0 .. gqa-1 of the 16-row tile), the softmax is fp32, the four warps' (m, l, O)
// are combined through shared memory, and the CTA leaves one partial per query head for
// merge_parts_kernel.  The whole step is a few microseconds of latency, not bandwidth: 2 052 keys
// are 4 MB.
constexpr int AM_WARPS = 4, AM_KEYS = 16 * AM_WARPS;
constexpr int AM_BOX = 16 * 128;                          // 16 keys x 64 dims bf16
constexpr int AM_OFF_K = 0, AM_OFF_V = AM_WARPS * 4 * AM_BOX, AM_OFF_Q = 2 * AM_WARPS * 4 * AM_BOX;
constexpr int AM_OFF_RED = AM_OFF_Q + 16 * 512, AM_OFF_M = AM_OFF_RED + 16 * RED_LD * 4, AM_OFF_L = AM_OFF_M + AM_WARPS * 16 * 4;
constexpr int AM_SMEM = AM_OFF_L + 16 * 4 + 1024;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    const int n = valid ? 16 : 0;                         // 0 bytes read: the 16 bytes arrive as zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

__global__ void __launch_bounds__(AM_WARPS * 32) attn_masked_mma_kernel(AttnSeq sq, int q_heads, int kv_heads, int gqa, float scale,
                                                                         const uint32_t *__restrict__ list, int list_stride,
                                                                         float *__restrict__ pacc, float *__restrict__ pstat) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *q_s = smem + AM_OFF_Q;
    float *red = reinterpret_cast<float *>(smem + AM_OFF_RED);
    float *sm_m = reinterpret_cast<float *>(smem + AM_OFF_M);
    float *sm_l = reinterpret_cast<float *>(smem + AM_OFF_L);
    const int chunk = blockIdx.x, h = blockIdx.y, r = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int n_rh = sq.rows * q_heads;
    const uint32_t *row_list = list + (size_t)r * list_stride;
    pdl_launch_next();
    pdl_wait();
    const int count = (int)min(row_list[0], (uint32_t)(list_stride - 1));
    const size_t part0 = ((size_t)chunk * n_rh + (size_t)r * q_heads + h * gqa) ;   // first of this CTA's gqa partial rows
    if (chunk * AM_KEYS >= count) {
        // nothing listed here: empty partials (sum 0 drops out of the merge)
        if (threadIdx.x < gqa) { pstat[(part0 + threadIdx.x) * 2] = -3.0e38f; pstat[(part0 + threadIdx.x) * 2 + 1] = 0.0f; }
        return;
    }
    // ---- gather: this warp's 16 keys
    const int e0 = chunk * AM_KEYS + warp * 16;
    uint32_t pos = 0xffffffffu;
    if (lane < 16 && e0 + lane < count) pos = row_list[1 + e0 + lane];
    const bool ok = pos < (uint32_t)sq.kc.max_ctx;
    int64_t kr = -1, vr = -1;
    if (ok) { kr = kv_row(sq.kc, h, (int)pos); vr = kv_row(sq.vc, h, (int)pos); }
    const uint32_t k_base = smem_u32(smem + AM_OFF_K + warp * 4 * AM_BOX), v_base = smem_u32(smem + AM_OFF_V + warp * 4 * AM_BOX);
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const int64_t kri = __shfl_sync(0xffffffffu, kr, i), vri = __shfl_sync(0xffffffffu, vr, i);
        const uint32_t off = (lane >> 3) * AM_BOX + swz128(i, (lane & 7) * 8);
        cp_async16(k_base + off, sq.kc.base + max(kri, (int64_t)0) * 256 + lane * 8, kri >= 0);
        cp_async16(v_base + off, sq.vc.base + max(vri, (int64_t)0) * 256 + lane * 8, vri >= 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const uint32_t valid = __ballot_sync(0xffffffffu, kr >= 0 && vr >= 0) & 0xffffu;     // bit i: key i of this warp counts
    // ---- Q of this (row, kv head): gqa rows of 256 fp32 -> bf16, swizzled (rows past gqa are zeros)
    for (int idx = threadIdx.x; idx < 16 * 32; idx += AM_WARPS * 32) {
        const int row = idx >> 5, ch = idx & 31;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (row < gqa) {
            const float *src = reinterpret_cast<const float *>(sq.q) + ((size_t)r * q_heads + h * gqa + row) * 256 + ch * 8;
            const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
            val.x = pack_bf16(a.x, a.y); val.y = pack_bf16(a.z, a.w); val.z = pack_bf16(b.x, b.y); val.w = pack_bf16(b.z, b.w);
        }
        *reinterpret_cast<uint4 *>(q_s + (ch >> 3) * AM_BOX + swz128(row, (ch & 7) * 8)) = val;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // ---- S = Q K^T for the warp's 16 keys
    const uint32_t q_base = smem_u32(q_s);
    const float sc2 = scale * LOG2E;
    float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    {
        const int mi = lane >> 3;
        const uint32_t q_row = (mi & 1) * 8 + (lane & 7), k_row = (mi >> 1) * 8 + (lane & 7);
#pragma unroll
        for (int ks = 0; ks < 16; ks++) {
            uint32_t a[4], b[4];
            const uint32_t qc = ks * 2 + (mi >> 1), kc = ks * 2 + (mi & 1);
            ldsm_x4(a[0], a[1], a[2], a[3], q_base + (qc >> 3) * AM_BOX + swz128(q_row, (qc & 7) * 8));
            ldsm_x4(b[0], b[1], b[2], b[3], k_base + (kc >> 3) * AM_BOX + swz128(k_row, (kc & 7) * 8));
            mma_bf16(s[0], a[0], a[1], a[2], a[3], b[0], b[1]);
            mma_bf16(s[1], a[0], a[1], a[2], a[3], b[2], b[3]);
        }
    }
    float m0, m1, l0, l1;
    uint32_t pa[4];
    {
#pragma unroll
        for (int n = 0; n < 2; n++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = n * 8 + tig * 2 + (e & 1);
                s[n][e] = (valid >> key & 1u) ? s[n][e] * sc2 : -INFINITY;
            }
        float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        m0 = fmaxf(mx0, NEG_BIG); m1 = fmaxf(mx1, NEG_BIG);
        const float p00 = ex2(s[0][0] - m0), p01 = ex2(s[0][1] - m0), p02 = ex2(s[0][2] - m1), p03 = ex2(s[0][3] - m1);
        const float p10 = ex2(s[1][0] - m0), p11 = ex2(s[1][1] - m0), p12 = ex2(s[1][2] - m1), p13 = ex2(s[1][3] - m1);
        l0 = (p00 + p01) + (p10 + p11); l1 = (p02 + p03) + (p12 + p13);
        pa[0] = pack_bf16(p00, p01); pa[1] = pack_bf16(p02, p03); pa[2] = pack_bf16(p10, p11); pa[3] = pack_bf16(p12, p13);
    }
    // ---- O = P V
    float o[32][4];
#pragma unroll
    for (int n = 0; n < 32; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    {
        const int mi = lane >> 3;
        const uint32_t v_row = (mi & 1) * 8 + (lane & 7);
#pragma unroll
        for (int np = 0; np < 16; np++) {
            uint32_t b[4];
            const uint32_t vc = np * 2 + (mi >> 1);
            ldsm_x4_t(b[0], b[1], b[2], b[3], v_base + (vc >> 3) * AM_BOX + swz128(v_row, (vc & 7) * 8));
            mma_bf16(o[np * 2], pa[0], pa[1], pa[2], pa[3], b[0], b[1]);
            mma_bf16(o[np * 2 + 1], pa[0], pa[1], pa[2], pa[3], b[2], b[3]);
        }
    }
    // ---- the four warps' (m, l, O) combined through shared memory, one round per warp
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (tig == 0) { sm_m[warp * 16 + gid] = m0; sm_m[warp * 16 + gid + 8] = m1; }
    __syncthreads();
    float M0 = NEG_BIG, M1 = NEG_BIG;
#pragma unroll
    for (int w = 0; w < AM_WARPS; w++) { M0 = fmaxf(M0, sm_m[w * 16 + gid]); M1 = fmaxf(M1, sm_m[w * 16 + gid + 8]); }
    {
        const float f0 = ex2(m0 - M0), f1 = ex2(m1 - M1);
        const bool v0 = gid < gqa, v1 = gid + 8 < gqa;
        float2 *r0 = reinterpret_cast<float2 *>(red + (size_t)gid * RED_LD + tig * 2);
        float2 *r1 = r0 + 8 * (RED_LD / 2);
#pragma unroll 1
        for (int round = 0; round < AM_WARPS; round++) {
            if (warp == round) {
                if (v0) {
#pragma unroll
                    for (int n = 0; n < 32; n++) {
                        const float2 t = round ? r0[n * 4] : make_float2(0.f, 0.f);
                        r0[n * 4] = make_float2(fmaf(o[n][0], f0, t.x), fmaf(o[n][1], f0, t.y));
                    }
                }
                if (v1) {
#pragma unroll
                    for (int n = 0; n < 32; n++) {
                        const float2 t = round ? r1[n * 4] : make_float2(0.f, 0.f);
                        r1[n * 4] = make_float2(fmaf(o[n][2], f1, t.x), fmaf(o[n][3], f1, t.y));
                    }
                }
                if (tig == 0) {
                    sm_l[gid] = (round ? sm_l[gid] : 0.0f) + l0 * f0;
                    sm_l[gid + 8] = (round ? sm_l[gid + 8] : 0.0f) + l1 * f1;
                }
            }
            __syncthreads();
        }
    }
    for (int idx = threadIdx.x; idx < gqa * 64; idx += AM_WARPS * 32) {
        const int row = idx >> 6, d4 = (idx & 63) * 4;
        float Mrow = NEG_BIG;
#pragma unroll
        for (int w = 0; w < AM_WARPS; w++) Mrow = fmaxf(Mrow, sm_m[w * 16 + row]);
        *reinterpret_cast<float4 *>(pacc + (part0 + row) * 256 + d4) = *reinterpret_cast<const float4 *>(red + (size_t)row * RED_LD + d4);
        if ((idx & 63) == 0) { pstat[(part0 + row) * 2] = Mrow * LN2; pstat[(part0 + row) * 2 + 1] = sm_l[row]; }
    }
}

// ---- per-query kernel: fp32 throughout (CUDA cores) ----------------------------------------
// The counterpart of the reference's qw_attn_decode (metal/attn.metal:32-129): no rounding
// of q or of the softmax weights, so it tracks the CPU twin to float rounding.  One block
// per (key slice, row, query head); 8 warps stride the slice's keys, a lane owns 8 dims.
// With a list (the QSA mask as positions, qwasar_gpu.h:635-645: per row a count, then that many
// positions ascending, list_stride uint32 apart) the "keys" are the list's entries, and only
// those positions of the cache are read; entries past the count are never touched, a position
// outside the cache is skipped.
__global__ void __launch_bounds__(256) attn_per_query_kernel(AttnSeq sq, int q_heads, int kv_heads, float scale,
                                                             float *pacc, float *pstat, int splits,
                                                             const uint32_t *__restrict__ list, int list_stride) {
    const int split = blockIdx.y, rh = blockIdx.x;
    const int r = rh / q_heads, h = rh - r * q_heads;
    const int kvh = h / (q_heads / kv_heads);
    const uint32_t *row_list = list ? list + (size_t)r * list_stride : nullptr;
    const int lo = list ? 0 : sq.key_lo;
    const int n = list ? (int)min(row_list[0], (uint32_t)(list_stride - 1)) : min(sq.key_hi, sq.base_pos + r + 1);
    const int per = max(1, (n - lo + splits - 1) / splits);
    const int t0 = lo + split * per, t1 = min(n, t0 + per);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float *qv = reinterpret_cast<const float *>(sq.q) + (size_t)rh * 256 + lane * 8;
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = qv[i] * scale;
    float m = -3.0e38f, l = 0.0f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = t0 + warp; j < t1; j += 8) {
        int t = j;
        if (row_list) {
            const uint32_t pos = row_list[1 + j];
            if (pos >= (uint32_t)sq.kc.max_ctx) continue;        // warp-uniform
            t = (int)pos;
        }
        const int64_t kr = kv_row(sq.kc, kvh, t), vr = kv_row(sq.vc, kvh, t);
        if (kr < 0 || vr < 0) continue;                          // a page that was never mapped
        const uint4 kk = reinterpret_cast<const uint4 *>(sq.kc.base + kr * 256)[lane];
        const uint4 vv = reinterpret_cast<const uint4 *>(sq.vc.base + vr * 256)[lane];
        const uint32_t kw[4] = {kk.x, kk.y, kk.z, kk.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            s += q[2 * i] * __uint_as_float(kw[i] << 16);
            s += q[2 * i + 1] * __uint_as_float(kw[i] & 0xffff0000u);
        }
        s = warp_sum(s);
        const float mn = fmaxf(m, s);
        const float a = expf(m - mn), pe = expf(s - mn);
        l = l * a + pe;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            acc[2 * i] = acc[2 * i] * a + pe * __uint_as_float(vw[i] << 16);
            acc[2 * i + 1] = acc[2 * i + 1] * a + pe * __uint_as_float(vw[i] & 0xffff0000u);
        }
        m = mn;
    }
    __shared__ float s_m[8], s_l[8], s_acc[8][256];
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < 8; i++) s_acc[warp][lane * 8 + i] = acc[i];
    __syncthreads();
    float M = -3.0e38f;
    for (int w = 0; w < 8; w++) if (s_l[w] > 0.0f) M = fmaxf(M, s_m[w]);
    float L = 0.0f, o = 0.0f;
    for (int w = 0; w < 8; w++) {
        const float f = s_l[w] > 0.0f ? expf(s_m[w] - M) : 0.0f;
        L += s_l[w] * f;
        o += s_acc[w][threadIdx.x] * f;
    }
    const size_t pi = (size_t)split * gridDim.x + rh;
    pacc[pi * 256 + threadIdx.x] = o;
    if (threadIdx.x == 0) { pstat[pi * 2] = M; pstat[pi * 2 + 1] = L; }
}

// Launch attribute of every kernel of the decode chain: it may start while the kernel in front of
// it on the stream still runs, and orders itself with pdl_wait() (qw_common.cuh).
void pdl_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute &attr, unsigned grid, unsigned block, size_t smem, cudaStream_t s) {
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg = cudaLaunchConfig_t();
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(block); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cfg.attrs = &attr; cfg.numAttrs = g_tune_pdl ? 1 : 0;
}

template <int MT, int KG>
void launch_split_t(cudaStream_t s, const AttnParams &p) {
    using Cfg = SplitCfg<MT, KG>;
    static bool configured[64] = {false};      // the attribute is per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(qw_attn_split_kernel<MT, KG>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    pdl_config(cfg, attr, (unsigned)p.n_cta, Cfg::THREADS, Cfg::SMEM, s);
    cudaLaunchKernelEx(&cfg, qw_attn_split_kernel<MT, KG>, p);
    g_launches++;
}

int row_tiles(int max_rows, int gqa) {
    const int need = (max_rows * gqa + 15) / 16;
    return need <= 1 ? 1 : (need <= 2 ? 2 : 4);
}

// ---- masked attention of one (row, KV head) on a CLUSTER: no partials in memory, no merge launch -------
// The row's list (at most a few thousand positions) is cut into steps of 16 keys, the steps dealt to the
// CTAs of a cluster and, inside a CTA, to its warps: a warp gathers its 16 K and V rows with asynchronous
// copies, computes S = Q K^T, the softmax weights and O = P V exactly as attn_masked_mma_kernel does, and
// keeps (max, sum, O) in registers over the steps it owns.  The warps of a CTA then add their O through
// the buffers the rows were gathered into, the CTAs add theirs through distributed shared memory -- each
// CTA finishes an equal slice of the output dims, gate included -- so the whole op is one launch and the
// only trips to memory are list -> rows -> output.  (As two launches with partials in between, the merge
// was 6 of the op's 17 us and the partials another trip.)
namespace cgx = cooperative_groups;
constexpr int AC_WARPS = 12;
constexpr int AC_OFF_KV = 0;                                   // per warp: K 8 KB | V 8 KB, later the warp's O [16][256] fp32
constexpr int AC_OFF_Q = AC_WARPS * 16384;                     // Q tile, bf16 [16][256] swizzled
constexpr int AC_OFF_ACC = AC_OFF_Q + 16 * 512;                // the CTA's O [16][256] fp32
constexpr int AC_OFF_M = AC_OFF_ACC + 16 * 1024;               // per warp row maxima [AC_WARPS][16]
constexpr int AC_OFF_L = AC_OFF_M + AC_WARPS * 64;             // per warp row sums   [AC_WARPS][16]
constexpr int AC_OFF_CM = AC_OFF_L + AC_WARPS * 64;            // the CTA's row maxima [16] and sums [16]
constexpr int AC_SMEM = AC_OFF_CM + 128 + 1024;
__global__ void __launch_bounds__(AC_WARPS * 32, 1)
attn_masked_cluster_kernel(AttnSeq sq, int q_heads, int kv_heads, int gqa, float scale, const uint32_t *__restrict__ list, int list_stride,
                           float *__restrict__ out, const float *__restrict__ gate, int gate_stride) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *q_s = smem + AC_OFF_Q;
    float *cta_acc = reinterpret_cast<float *>(smem + AC_OFF_ACC);
    float *sm_m = reinterpret_cast<float *>(smem + AC_OFF_M), *sm_l = reinterpret_cast<float *>(smem + AC_OFF_L);
    float *cta_ml = reinterpret_cast<float *>(smem + AC_OFF_CM);
    cgx::cluster_group cluster = cgx::this_cluster();
    const int C = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int h = blockIdx.y, r = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const uint32_t *row_list = list + (size_t)r * list_stride;
    pdl_launch_next();
    pdl_wait();
    // the count and the first step's positions are asked for together (entries past the count are inside the
    // row of the list and simply not used): one trip to memory instead of two
    const int guess = (rank * AC_WARPS + warp) * 16 + lane;      // where this lane's first key sits if the list is full
    uint32_t pos_guess = 0xffffffffu;
    if (lane < 16 && guess < list_stride - 1) pos_guess = __ldg(row_list + 1 + guess);
    const int count = (int)min(__ldg(row_list), (uint32_t)(list_stride - 1));
    const int steps = (count + 15) >> 4, spc = (steps + C - 1) / C;   // steps per CTA
    const int s0 = min(rank * spc, steps), s1 = min(s0 + spc, steps);

    // ---- Q of this (row, kv head): gqa rows of 256 fp32 -> bf16, swizzled (rows past gqa are zeros)
    for (int idx = threadIdx.x; idx < 16 * 32; idx += AC_WARPS * 32) {
        const int row = idx >> 5, ch = idx & 31;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (row < gqa) {
            const float *src = reinterpret_cast<const float *>(sq.q) + ((size_t)r * q_heads + h * gqa + row) * 256 + ch * 8;
            const float4 a = __ldg(reinterpret_cast<const float4 *>(src)), b = __ldg(reinterpret_cast<const float4 *>(src + 4));
            val.x = pack_bf16(a.x, a.y); val.y = pack_bf16(a.z, a.w); val.z = pack_bf16(b.x, b.y); val.w = pack_bf16(b.z, b.w);
        }
        *reinterpret_cast<uint4 *>(q_s + (ch >> 3) * AM_BOX + swz128(row, (ch & 7) * 8)) = val;
    }
    __syncthreads();

    const uint32_t k_base = smem_u32(smem + AC_OFF_KV + warp * 16384), v_base = k_base + 4 * AM_BOX;
    const uint32_t q_base = smem_u32(q_s);
    const float sc2 = scale * LOG2E;
    float o[32][4];
#pragma unroll
    for (int n = 0; n < 32; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    float m0 = NEG_BIG, m1 = NEG_BIG, l0 = 0.0f, l1 = 0.0f;
    for (int st = s0 + warp; st < s1; st += AC_WARPS) {
        // ---- gather: 16 keys
        const int e0 = st * 16;
        uint32_t pos = 0xffffffffu;
        if (lane < 16 && e0 + lane < count) pos = (e0 + lane == guess) ? pos_guess : __ldg(row_list + 1 + e0 + lane);
        const bool ok = pos < (uint32_t)sq.kc.max_ctx;
        int kr = -1, vr = -1;                                   // rows of the cache arrays (below 2^31: 512 bytes each)
        if (ok) { kr = (int)kv_row(sq.kc, h, (int)pos); vr = (int)kv_row(sq.vc, h, (int)pos); }
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int kri = __shfl_sync(0xffffffffu, kr, i), vri = __shfl_sync(0xffffffffu, vr, i);
            const uint32_t off = (lane >> 3) * AM_BOX + swz128(i, (lane & 7) * 8);
            cp_async16(k_base + off, sq.kc.base + (size_t)max(kri, 0) * 256 + lane * 8, kri >= 0);
            cp_async16(v_base + off, sq.vc.base + (size_t)max(vri, 0) * 256 + lane * 8, vri >= 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        const uint32_t valid = __ballot_sync(0xffffffffu, kr >= 0 && vr >= 0) & 0xffffu;     // bit i: key i counts
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        // ---- S = Q K^T
        float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
        {
            const int mi = lane >> 3;
            const uint32_t q_row = (mi & 1) * 8 + (lane & 7), k_row = (mi >> 1) * 8 + (lane & 7);
#pragma unroll
            for (int ks = 0; ks < 16; ks++) {
                uint32_t a[4], b[4];
                const uint32_t qc = ks * 2 + (mi >> 1), kc = ks * 2 + (mi & 1);
                ldsm_x4(a[0], a[1], a[2], a[3], q_base + (qc >> 3) * AM_BOX + swz128(q_row, (qc & 7) * 8));
                ldsm_x4(b[0], b[1], b[2], b[3], k_base + (kc >> 3) * AM_BOX + swz128(k_row, (kc & 7) * 8));
                mma_bf16(s[0], a[0], a[1], a[2], a[3], b[0], b[1]);
                mma_bf16(s[1], a[0], a[1], a[2], a[3], b[2], b[3]);
            }
        }
        uint32_t pa[4];
        {
#pragma unroll
            for (int n = 0; n < 2; n++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int key = n * 8 + tig * 2 + (e & 1);
                    s[n][e] = (valid >> key & 1u) ? s[n][e] * sc2 : -INFINITY;
                }
            float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
            float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
            if (st != s0 + warp) {                              // a later step of this warp: what it holds moves to the new maxima
                const float f0 = ex2(m0 - n0), f1 = ex2(m1 - n1);
                l0 *= f0; l1 *= f1;
#pragma unroll
                for (int n = 0; n < 32; n++) { o[n][0] *= f0; o[n][1] *= f0; o[n][2] *= f1; o[n][3] *= f1; }
            }
            m0 = n0; m1 = n1;
            const float p00 = ex2(s[0][0] - m0), p01 = ex2(s[0][1] - m0), p02 = ex2(s[0][2] - m1), p03 = ex2(s[0][3] - m1);
            const float p10 = ex2(s[1][0] - m0), p11 = ex2(s[1][1] - m0), p12 = ex2(s[1][2] - m1), p13 = ex2(s[1][3] - m1);
            l0 += (p00 + p01) + (p10 + p11); l1 += (p02 + p03) + (p12 + p13);
            pa[0] = pack_bf16(p00, p01); pa[1] = pack_bf16(p02, p03); pa[2] = pack_bf16(p10, p11); pa[3] = pack_bf16(p12, p13);
        }
        // ---- O += P V
        {
            const int mi = lane >> 3;
            const uint32_t v_row = (mi & 1) * 8 + (lane & 7);
#pragma unroll
            for (int np = 0; np < 16; np++) {
                uint32_t b[4];
                const uint32_t vc = np * 2 + (mi >> 1);
                ldsm_x4_t(b[0], b[1], b[2], b[3], v_base + (vc >> 3) * AM_BOX + swz128(v_row, (vc & 7) * 8));
                mma_bf16(o[np * 2], pa[0], pa[1], pa[2], pa[3], b[0], b[1]);
                mma_bf16(o[np * 2 + 1], pa[0], pa[1], pa[2], pa[3], b[2], b[3]);
            }
        }
        __syncwarp();                                           // the buffer may be gathered into again
    }
    // ---- the CTA's warps add up: maxima first, then every warp leaves its O, moved to the CTA's maxima, in its buffer
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (tig == 0) { sm_m[warp * 16 + gid] = m0; sm_m[warp * 16 + gid + 8] = m1; }
    __syncthreads();
    float M0 = NEG_BIG, M1 = NEG_BIG;
#pragma unroll
    for (int w = 0; w < AC_WARPS; w++) { M0 = fmaxf(M0, sm_m[w * 16 + gid]); M1 = fmaxf(M1, sm_m[w * 16 + gid + 8]); }
    const bool has_steps = s0 + warp < s1;
    {
        const float f0 = ex2(m0 - M0), f1 = ex2(m1 - M1);
        if (tig == 0) { sm_l[warp * 16 + gid] = l0 * f0; sm_l[warp * 16 + gid + 8] = l1 * f1; }
        if (has_steps) {
            // [16 rows][128 float2], the float2 index xor-ed with (row & 3) << 2: the eight rows of a store then
            // meet no more bank conflicts than 256 bytes per request cost anyway
            float2 *w_o = reinterpret_cast<float2 *>(smem + AC_OFF_KV + warp * 16384);
            const int x0 = (gid & 3) << 2;
            if (gid < gqa) {                                    // (only the rows that exist: this phase is shared-memory bandwidth)
#pragma unroll
                for (int n = 0; n < 32; n++) w_o[gid * 128 + ((n * 4 + tig) ^ x0)] = make_float2(o[n][0] * f0, o[n][1] * f0);
            }
            if (gid + 8 < gqa) {
#pragma unroll
                for (int n = 0; n < 32; n++) w_o[(gid + 8) * 128 + ((n * 4 + tig) ^ x0)] = make_float2(o[n][2] * f1, o[n][3] * f1);
            }
        }
    }
    __syncthreads();
    const int live_warps = min(AC_WARPS, max(s1 - s0, 0));       // warps 0 .. live_warps - 1 hold something
    for (int idx = threadIdx.x; idx < gqa * 64; idx += AC_WARPS * 32) {
        const int row = idx >> 6, c4 = idx & 63;
        const int p4 = c4 ^ ((row & 3) << 1);                    // (the float2 swizzle, in float4 units)
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int w = 0; w < live_warps; w++) {
            const float4 a = *reinterpret_cast<const float4 *>(smem + AC_OFF_KV + w * 16384 + (row * 64 + p4) * 16);
            acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
        }
        *reinterpret_cast<float4 *>(cta_acc + row * 256 + c4 * 4) = acc;
    }
    if (threadIdx.x < 16) {
        float mm = NEG_BIG, ll = 0.0f;
        for (int w = 0; w < AC_WARPS; w++) { mm = fmaxf(mm, sm_m[w * 16 + threadIdx.x]); ll += sm_l[w * 16 + threadIdx.x]; }
        cta_ml[threadIdx.x] = mm; cta_ml[16 + threadIdx.x] = ll;
    }
    cluster.sync();                                             // every CTA's (max, sum, O) is in its shared memory
    // ---- the cluster adds up: CTA `rank` finishes its slice of the gqa x 64 float4 of the output
    {
        const int total = gqa * 64, per = (total + C - 1) / C;
        const int idx = rank * per + threadIdx.x;
        if (threadIdx.x < per && idx < total) {
            const int row = idx >> 6, c4 = idx & 63;
            // all remote reads are issued before the first is used (one after the other they were 2 x C round trips
            // between SMs on the op's critical path)
            float mq[16], lq[16];
            float4 aq[16];
#pragma unroll
            for (int q = 0; q < 16; q++) {
                mq[q] = NEG_BIG; lq[q] = 0.0f; aq[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (q < C) {
                    const float *ml = cluster.map_shared_rank(cta_ml, q);
                    mq[q] = ml[row]; lq[q] = ml[16 + row];
                    aq[q] = *reinterpret_cast<const float4 *>(cluster.map_shared_rank(cta_acc, q) + row * 256 + c4 * 4);
                }
            }
            float M = NEG_BIG;
#pragma unroll
            for (int q = 0; q < 16; q++) M = fmaxf(M, mq[q]);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float den = 0.0f;
#pragma unroll
            for (int q = 0; q < 16; q++) {
                const float f = ex2(mq[q] - M);
                acc.x = fmaf(aq[q].x, f, acc.x); acc.y = fmaf(aq[q].y, f, acc.y); acc.z = fmaf(aq[q].z, f, acc.z); acc.w = fmaf(aq[q].w, f, acc.w);
                den = fmaf(lq[q], f, den);
            }
            const float inv = den > 0.0f ? 1.0f / den : 0.0f;
            acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
            const size_t rh = (size_t)r * q_heads + h * gqa + row;
            if (gate) {
                const float4 g = __ldg(reinterpret_cast<const float4 *>(gate + rh * gate_stride + c4 * 4));
                acc.x *= sigmoidf(g.x); acc.y *= sigmoidf(g.y); acc.z *= sigmoidf(g.z); acc.w *= sigmoidf(g.w);
            }
            *reinterpret_cast<float4 *>(out + rh * 256 + c4 * 4) = acc;
        }
    }
    cluster.sync();                                             // no CTA leaves while another may still read its shared memory
}

}  // namespace

unsigned long long g_launches = 0;
int g_tune_split_kg = 6;
int g_tune_prefill_tc = 1;
int g_tune_prefill_fuse_q = 1;
int g_tune_pdl = 1;
int g_tune_masked_tc = 1;
int g_tune_qmv_tc = 1;
int g_tune_split_kg2 = 3;
int g_tune_qmv_pre = 1;

int sm_count() {
    static int n[64] = {0};                    // per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 148;
    if (!n[dev]) {
        cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
        if (n[dev] <= 0) n[dev] = 148;
    }
    return n[dev];
}

size_t attn_split_scratch_bytes(const AttnParams &p, int max_rows) {
    const int mt = row_tiles(max_rows, p.gqa);
    size_t rows_total = 0;
    for (int i = 0; i < p.n_seq; i++) rows_total += p.seq[i].rows;
    // slots, then (mode 1) one combined partial per (row, head)
    return ((size_t)attn_split_slots(p) * mt * 16 + rows_total * p.q_heads) * 258 * sizeof(float);
}

void launch_attn_split(cudaStream_t s, const AttnParams &p, int max_rows) {
    switch (row_tiles(max_rows, p.gqa)) {
        case 1:
            if (g_tune_split_kg == 4) launch_split_t<1, 4>(s, p);
            else launch_split_t<1, 6>(s, p);
            break;
        case 2:
            if (g_tune_split_kg2 == 3) launch_split_t<2, 3>(s, p);
            else launch_split_t<2, 2>(s, p);
            break;
        default: launch_split_t<4, 1>(s, p); break;
    }
}

// The cut of the tile line, for the host: first tile of every CTA's share (n_cta + 1 entries).
void attn_split_shares(const AttnParams &p, int32_t *share_first) {
    for (int c = 0; c <= p.n_cta; c++) share_first[c] = share_lo(p, c);
}
// Whether any group of the launch is cut over more than one CTA (its output then comes from the merge).
bool attn_split_needs_merge(const AttnParams &p) {
    for (int i = 0; i < p.n_seq; i++)
        for (int h = 0; h < p.kv_heads; h++) {
            const int64_t g0 = (int64_t)p.seq[i].cum_tiles + (int64_t)h * p.seq[i].n_tiles;
            int c0, c1;
            group_ctas(p, g0, g0 + p.seq[i].n_tiles, c0, c1);
            if (c0 != c1) return true;
        }
    return false;
}

void launch_attn_merge(cudaStream_t s, const AttnParams &p, int max_rows) {
    const int vr = max_rows * p.gqa;
    const unsigned blocks = (unsigned)(p.n_seq * p.kv_heads * vr);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    pdl_config(cfg, attr, blocks, MERGE_THREADS, 0, s);
    switch (row_tiles(max_rows, p.gqa)) {
        case 1: cudaLaunchKernelEx(&cfg, qw_attn_merge_kernel<1>, p, vr); break;
        case 2: cudaLaunchKernelEx(&cfg, qw_attn_merge_kernel<2>, p, vr); break;
        default: cudaLaunchKernelEx(&cfg, qw_attn_merge_kernel<4>, p, vr); break;
    }
    g_launches++;
}

void launch_merge_parts(cudaStream_t s, void *out, int out_dtype, const float *pacc, const float *pstat,
                        const void *gate, int gate_dtype, int gate_stride, int n_rows_heads, int parts,
                        float *pacc_out, float *pstat_out, size_t acc_stride, size_t stat_stride) {
    if (n_rows_heads <= 0) return;
    if (!acc_stride) acc_stride = (size_t)n_rows_heads * 256;
    if (!stat_stride) stat_stride = (size_t)n_rows_heads * 2;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    pdl_config(cfg, attr, (unsigned)n_rows_heads, 256, (size_t)parts * sizeof(float), s);
    cudaLaunchKernelEx(&cfg, merge_parts_kernel, out, out_dtype, pacc, pstat, gate, gate_dtype, gate_stride, n_rows_heads, parts,
                       pacc_out, pstat_out, acc_stride, stat_stride);
    g_launches++;
}

// Masked attention of `rows` rows over their position lists on tensor ops: n_chunks = ceil(cap / 64)
// partials per (row, head) into pacc [n_chunks, rows * q_heads, 256] / pstat, for launch_merge_parts.
int attn_masked_chunks(int cap) { return (cap + AM_KEYS - 1) / AM_KEYS; }
// The cluster form of the masked attention (fp32 rows in and out, at most 16 q heads per KV head); false where it
// does not apply or a cluster cannot be placed, and the caller then takes the two-launch path.
bool launch_attn_masked_cluster(cudaStream_t s, const AttnSeq &seq, int q_heads, int kv_heads, float scale, const uint32_t *list,
                                int list_stride, float *out, const float *gate, int gate_stride) {
    static int cluster_size[64] = {0};                          // per device: 0 not tried, -1 unavailable, else CTAs per cluster
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return false;
    const int gqa = q_heads / kv_heads;
    if (gqa > 16 || (gate && ((reinterpret_cast<uintptr_t>(gate) & 15) || (gate_stride & 3)))) return false;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    cfg.blockDim = dim3(AC_WARPS * 32); cfg.dynamicSmemBytes = AC_SMEM; cfg.stream = s;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    if (cluster_size[dev] == 0) {
        cluster_size[dev] = -1;
        if (cudaFuncSetAttribute(attn_masked_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AC_SMEM) == cudaSuccess) {
            cudaFuncSetAttribute(attn_masked_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            for (int c : {16, 8}) {                             // the largest cluster this device can place
                int n = 0;
                cfg.gridDim = dim3(c, 1, 1); attr[0].val.clusterDim.x = c; cfg.numAttrs = 1;
                if (cudaOccupancyMaxActiveClusters(&n, attn_masked_cluster_kernel, &cfg) == cudaSuccess && n >= 1) { cluster_size[dev] = c; break; }
            }
            cudaGetLastError();
        }
    }
    const int C = cluster_size[dev];
    if (C <= 0) return false;
    cfg.gridDim = dim3((unsigned)C, (unsigned)kv_heads, (unsigned)seq.rows);
    attr[0].val.clusterDim.x = C;
    cfg.numAttrs = g_tune_pdl ? 2 : 1;
    if (cudaLaunchKernelEx(&cfg, attn_masked_cluster_kernel, seq, q_heads, kv_heads, gqa, scale, list, list_stride, out, gate, gate_stride) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    g_launches++;
    return true;
}


void launch_attn_masked_mma(cudaStream_t s, const AttnSeq &seq, int q_heads, int kv_heads, float scale, const uint32_t *list,
                            int list_stride, float *pacc, float *pstat) {
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(attn_masked_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AM_SMEM);
        configured[dev] = true;
    }
    const int gqa = q_heads / kv_heads;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    pdl_config(cfg, attr, 1, AM_WARPS * 32, AM_SMEM, s);
    cfg.gridDim = dim3((unsigned)attn_masked_chunks(list_stride - 1), (unsigned)kv_heads, (unsigned)seq.rows);
    cudaLaunchKernelEx(&cfg, attn_masked_mma_kernel, seq, q_heads, kv_heads, gqa, scale, list, list_stride, pacc, pstat);
    g_launches++;
}

int attn_per_query_splits(int rows, int q_heads, int n_keys) {
    int want = (2 * sm_count() + rows * q_heads - 1) / (rows * q_heads);
    int cap = (n_keys + 255) / 256;
    return std::max(1, std::min(want, cap));
}
size_t attn_per_query_scratch_bytes(int rows, int q_heads, int splits) {
    return (size_t)splits * rows * q_heads * 258 * sizeof(float);
}
void launch_attn_per_query(cudaStream_t s, const AttnSeq &seq, int q_heads, int kv_heads, float scale, float *pacc,
                           float *pstat, int splits, const uint32_t *list, int list_stride) {
    dim3 grid(seq.rows * q_heads, splits);
    attn_per_query_kernel<<<grid, 256, 0, s>>>(seq, q_heads, kv_heads, scale, pacc, pstat, splits, list, list_stride);
    g_launches++;
}

}  // namespace qw
