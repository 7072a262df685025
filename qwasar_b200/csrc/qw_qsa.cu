// QSA's indexer on the device: block keys, block scores and the top-k selection that turns scores
// into the byte mask and the position list which qw_op_attn_masked walks (qwasar_gpu.h:620-639;
// the CPU statement is qsa_select, qwasar_flash_cpu.c:345-418).
//
//   block key b   = rope(rms_norm(mean of the ratio raw index keys of block b) * k_norm) at position b * ratio
//   score(r, b)   = sum over the nq index heads of max(qn[r, h] . key_b, 0) / sqrt(d),  b < (base_pos + r + 1) / ratio
//   selection     = the block_topk best complete blocks, found one at a time (largest score above
//                   -FLT_MAX, lowest index among equals), plus the incomplete trailing block
//
// The arithmetic of a block key is written once (block_key) and used by both the pooling op and
// the scoring-from-raw-keys op, so scores from stored block keys are identical to scores from raw
// keys (the reference tests that equality, tests/test_sparse.c:372-391).  Operation order follows
// the CPU statement except for the 256-term sums, which are warp reductions; contraction is off
// through the _rn intrinsics.  These are small kernels: first correct versions, not tuned.
#include <float.h>
#include <algorithm>
#include <cooperative_groups.h>

#include "qw_kernels.h"

namespace qw {

namespace {

// Lane l holds dims l + 32 k (k < d / 32 <= 8), so that the RoPE pair (j, j + 32), j < 32, sits in
// one lane (rotary_dim == 64).
__device__ __forceinline__ void block_key(float (&x)[8], const float *__restrict__ ikeys, const uint16_t *__restrict__ k_norm,
                                          const float *__restrict__ inv_freq, int d, int ratio, int b, float eps, int lane) {
    const int nk = d >> 5;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        x[k] = 0.0f;
        if (k < nk) {
            float acc = 0.0f;
            for (int t = 0; t < ratio; t++) acc = __fadd_rn(acc, ikeys[(size_t)(b * ratio + t) * d + lane + 32 * k]);
            x[k] = __fdiv_rn(acc, (float)ratio);
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; k++) ss = __fadd_rn(ss, __fmul_rn(x[k], x[k]));
    ss = warp_sum(ss);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)d), eps)));
#pragma unroll
    for (int k = 0; k < 8; k++) {
        if (k < nk) {
            x[k] = __fmul_rn(x[k], inv);
            if (k_norm) x[k] = __fmul_rn(x[k], bf16_bits_to_f32(k_norm[lane + 32 * k]));
        }
    }
    const float ang = __fmul_rn((float)(b * ratio), inv_freq[lane]);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    const float lo = x[0], hi = x[1];
    x[0] = __fsub_rn(__fmul_rn(lo, cs), __fmul_rn(hi, sn));
    x[1] = __fadd_rn(__fmul_rn(hi, cs), __fmul_rn(lo, sn));
}

// one warp per block b0 + ...
__global__ void __launch_bounds__(256) qsa_pool_kernel(float *__restrict__ pool, const float *__restrict__ ikeys,
                                                       const uint16_t *__restrict__ k_norm, const float *__restrict__ inv_freq,
                                                       int d, int ratio, int b0, int b1, float eps) {
    const int b = b0 + blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (b >= b1) return;
    float x[8];
    block_key(x, ikeys, k_norm, inv_freq, d, ratio, b, eps, lane);
#pragma unroll
    for (int k = 0; k < 8; k++)
        if (k < (d >> 5)) pool[(size_t)b * d + lane + 32 * k] = x[k];
}

// one warp per (row, block): grid (ceil(max visible blocks / 8), rows)
__global__ void __launch_bounds__(256) qsa_scores_kernel(float *__restrict__ scores, const float *__restrict__ qn,
                                                         const float *__restrict__ pool, int nq, int d, int ratio, int base_pos,
                                                         int max_blocks) {
    const int r = blockIdx.y, b = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int n_blocks = (base_pos + r + 1) / ratio;
    if (b >= n_blocks || b >= max_blocks) return;
    const int nk = d >> 5;
    float key[8];
#pragma unroll
    for (int k = 0; k < 8; k++) key[k] = k < nk ? pool[(size_t)b * d + lane + 32 * k] : 0.0f;
    float s = 0.0f;
    for (int h = 0; h < nq; h++) {
        const float *q = qn + ((size_t)r * nq + h) * d;
        float dot = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; k++)
            if (k < nk) dot = __fadd_rn(dot, __fmul_rn(q[lane + 32 * k], key[k]));
        dot = warp_sum(dot);
        if (dot > 0.0f) s = __fadd_rn(s, dot);
    }
    if (lane == 0) scores[(size_t)r * max_blocks + b] = __fdiv_rn(s, sqrtf((float)d));
}

// One CTA per row.  The reference finds the block_topk best blocks one at a time (the largest score
// above -FLT_MAX, the lowest index among equals): that is the first `take` blocks in the order
// (score descending, index ascending).  Found here without sorting: the scores map to unsigned
// keys that order the same way (-0 and +0 share a key, as they compare equal), a radix select of
// four 8-bit passes finds the key of the take-th best, every block with a larger key is taken, and
// of the blocks with exactly that key the lowest-indexed ones until the count is reached.  Every
// sweep reads the row with consecutive lanes on consecutive scores (a warp whose lanes each walk a
// run of their own costs one cache-line look-up per lane and load, which was the whole run time).
// The two ordered sweeps give every warp one contiguous stretch of blocks; ballots rank the equals
// and place the taken blocks inside each group of 32.
// SEL_BATCH loads are in flight per thread before the first is used: the branches and the
// shared-memory updates of a sweep otherwise keep the compiler from overlapping them.
constexpr int SEL_THREADS = 1024, SEL_WARPS = SEL_THREADS / 32, SEL_BATCH = 8;
__device__ __forceinline__ bool sel_key(float v, uint32_t &key) {
    if (!(v > -FLT_MAX)) return false;                            // -FLT_MAX, -inf and NaN are never selected
    if (v == 0.0f) v = 0.0f;                                      // -0 -> +0
    const uint32_t u = __float_as_uint(v);
    key = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return true;
}
__global__ void __launch_bounds__(SEL_THREADS) qsa_select_kernel(uint8_t *__restrict__ mask, uint32_t *__restrict__ list,
                                                                 const float *__restrict__ scores, int ratio, int base_pos,
                                                                 int block_topk, int max_ctx, int max_blocks, int list_stride) {
    __shared__ int hist[256];
    __shared__ int w_gt[SEL_WARPS], w_eq[SEL_WARPS];
    __shared__ uint32_t s_prefix;
    __shared__ int s_remaining, s_take, s_total;
    const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t below = (1u << lane) - 1u;
    const int n_keys = base_pos + r + 1, n_blocks = n_keys / ratio;
    const float *sc = scores + (size_t)r * max_blocks;
    uint8_t *m = mask + (size_t)r * max_ctx;
    uint32_t *l = list + (size_t)r * list_stride;
    // the mask starts as 0 over the blocks and 1 over the tail; 16 bytes per store where the row allows
    const int tail0 = n_blocks * ratio;
    const int head = min((int)((16 - ((uintptr_t)m & 15)) & 15), n_keys);
    const int vec_end = tail0 > head ? head + ((tail0 - head) & ~15) : head;
    for (int t = tid; t < head; t += SEL_THREADS) m[t] = t >= tail0;
    for (int t = head + 16 * tid; t < vec_end; t += 16 * SEL_THREADS) *reinterpret_cast<uint4 *>(m + t) = make_uint4(0, 0, 0, 0);
    for (int t = vec_end + tid; t < n_keys; t += SEL_THREADS) m[t] = t >= tail0;
    if (tid == 0) { s_prefix = 0; s_remaining = 0; s_take = 0; }

    // radix select: after the pass over byte `shift`, s_prefix holds the top bytes of the key of
    // the take-th best block and s_remaining how many blocks with that prefix are still wanted.
    // The first pass sees every block that can be selected at all, which fixes `take`.
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix, high = shift == 24 ? 0u : 0xFFFFFFFFu << (shift + 8);
        // scores of one row mostly share their top bytes: count a run of one bin in a register
        // and add it once, or the whole row queues up on one shared-memory word
        int cur = 0, run = 0;
        for (int b0 = tid; b0 < n_blocks; b0 += SEL_BATCH * SEL_THREADS) {
            float v[SEL_BATCH];
#pragma unroll
            for (int j = 0; j < SEL_BATCH; j++) {
                const int b = b0 + j * SEL_THREADS;
                v[j] = b < n_blocks ? sc[b] : -FLT_MAX;
            }
#pragma unroll
            for (int j = 0; j < SEL_BATCH; j++) {
                uint32_t key;
                if (!(sel_key(v[j], key) && (key & high) == prefix)) continue;
                const int bin = (key >> shift) & 0xFF;
                if (bin == cur) { run++; continue; }
                if (run) atomicAdd(&hist[cur], run);
                cur = bin; run = 1;
            }
        }
        if (run) atomicAdd(&hist[cur], run);
        __syncthreads();
        // Walking down from bin 255, the first bin at which the count reaches `want` (bin 0 if none
        // does) holds the key looked for.  One warp: lane l sums bins 255-8l .. 248-8l, a scan over
        // the lanes finds the lane in whose bins the count is reached, that lane walks its eight.
        if (warp == 0) {
            int want = s_remaining;
            __syncwarp();
            int h[8], mine = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) { h[j] = hist[255 - 8 * lane - j]; mine += h[j]; }
            int incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const int all = __shfl_sync(0xffffffffu, incl, 31);
            if (shift == 24) {
                want = min(min(block_topk, n_blocks), all);       // every block that can be selected is in this histogram
                if (lane == 0) s_take = want;
            }
            const uint32_t reached = __ballot_sync(0xffffffffu, incl >= want);
            if (reached == 0u) {
                if (lane == 31) { s_remaining = want - (all - h[7]); s_prefix = prefix; }   // bin 0
            } else if (lane == __ffs(reached) - 1) {
                int run = incl - mine, bin = 0, rem = 0;
                bool done = false;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (!done && (run + h[j] >= want || 8 * lane + j == 255)) { bin = 255 - 8 * lane - j; rem = want - run; done = true; }
                    run += h[j];
                }
                s_remaining = rem;                                // still wanted among the keys of this bin
                s_prefix = prefix | ((uint32_t)bin << shift);
            }
        }
        __syncthreads();
        if (s_take <= 0) break;
    }
    const int take = s_take;
    const uint32_t kth = s_prefix;                                // the key of the take-th best block
    const int need_eq = s_remaining;                              // blocks with exactly that key to take, lowest index first

    // this warp's stretch of blocks, a multiple of 32 long
    const int chunk = (n_blocks + SEL_THREADS - 1) / SEL_THREADS * 32;
    const int w_lo = min(warp * chunk, n_blocks), w_hi = min(w_lo + chunk, n_blocks);
    int gt = 0, eq = 0;
    if (take > 0)
        for (int b0 = w_lo + lane; b0 < w_hi; b0 += SEL_BATCH * 32) {
            float v[SEL_BATCH];
#pragma unroll
            for (int j = 0; j < SEL_BATCH; j++) {
                const int b = b0 + j * 32;
                v[j] = b < w_hi ? sc[b] : -FLT_MAX;
            }
#pragma unroll
            for (int j = 0; j < SEL_BATCH; j++) {
                uint32_t key;
                if (sel_key(v[j], key)) { gt += key > kth; eq += key == kth; }
            }
        }
    gt = (int)__reduce_add_sync(0xffffffffu, (unsigned)gt);
    eq = (int)__reduce_add_sync(0xffffffffu, (unsigned)eq);
    if (lane == 0) { w_gt[warp] = gt; w_eq[warp] = eq; }
    __syncthreads();
    if (tid == 0) {                                               // per warp: equals before it, taken blocks before it
        int eq_run = 0, out_run = 0;
        for (int w = 0; w < SEL_WARPS; w++) {
            const int e = w_eq[w], g = w_gt[w];
            w_eq[w] = eq_run; w_gt[w] = out_run;
            out_run += g + min(max(need_eq - eq_run, 0), e);
            eq_run += e;
        }
        s_total = out_run;                                        // blocks taken in all (== take)
    }
    __syncthreads();
    // the mask of the taken blocks, and the list: taken blocks in ascending order, then the tail
    if (take > 0) {
        int eq_rank = w_eq[warp], at = w_gt[warp];
        for (int b0 = w_lo + lane; b0 < w_hi + lane; b0 += SEL_BATCH * 32) {   // the same trip count on every lane
            float v[SEL_BATCH];
#pragma unroll
            for (int j = 0; j < SEL_BATCH; j++) {
                const int b = b0 + j * 32;
                v[j] = b < w_hi ? sc[b] : -FLT_MAX;
            }
#pragma unroll
            for (int j = 0; j < SEL_BATCH; j++) {
                const int b = b0 + j * 32;
                bool is_gt = false, is_eq = false;
                uint32_t key;
                if (sel_key(v[j], key)) { is_gt = key > kth; is_eq = key == kth; }
                const uint32_t eq_bits = __ballot_sync(0xffffffffu, is_eq);
                const bool taken = is_gt || (is_eq && eq_rank + __popc(eq_bits & below) < need_eq);
                const uint32_t t_bits = __ballot_sync(0xffffffffu, taken);
                if (taken) {
                    const int pos = (at + __popc(t_bits & below)) * ratio;
                    for (int t = 0; t < ratio; t++) {
                        m[b * ratio + t] = 1;
                        l[1 + pos + t] = (uint32_t)(b * ratio + t);
                    }
                }
                eq_rank += __popc(eq_bits);
                at += __popc(t_bits);
            }
        }
    }
    const int total = s_total * ratio;
    for (int t = tail0 + tid; t < n_keys; t += SEL_THREADS) l[1 + total + (t - tail0)] = (uint32_t)t;
    if (tid == 0) l[0] = (uint32_t)(total + (n_keys - tail0));
}


// ---- the selection of a long row, spread over a cluster of eight CTAs --------------------------------
// The same selection as qsa_select_kernel (same keys, same radix select, same order of the list),
// for rows of thousands of blocks, where one CTA sweeping the row six times from L2 is all latency:
// 65 536 scores took 67 us.  Here a cluster of SC_CTAS CTAs (distributed shared memory) takes one row;
// CTA q reads its contiguous share of the scores ONCE, as order-preserving keys into shared memory
// (0 = not selectable), and every later pass runs from there.  A radix pass builds a 256-bin
// histogram per CTA (warp-aggregated adds), the cluster synchronises, every CTA sums the eight
// histograms through distributed shared memory and takes the same decision; the ordered passes need
// only each CTA's counts of larger and equal keys, read the same way.  The mask is cleared and the
// list written by the CTAs in parallel, each for its own stretch of blocks.
namespace cg = cooperative_groups;
constexpr int SC_CTAS = 8, SC_THREADS = 1024, SC_WARPS = SC_THREADS / 32;

__global__ void __cluster_dims__(SC_CTAS, 1, 1) __launch_bounds__(SC_THREADS)
qsa_select_cluster_kernel(uint8_t *__restrict__ mask, uint32_t *__restrict__ list, const float *__restrict__ scores, int ratio,
                          int base_pos, int block_topk, int max_ctx, int max_blocks, int list_stride, int per_cta) {
    extern __shared__ uint32_t keys[];                            // per_cta keys of this CTA's blocks
    __shared__ int hist[256];
    __shared__ int tot[256];
    __shared__ int w_gt[SC_WARPS], w_eq[SC_WARPS];
    __shared__ int cta_cnt[2];                                    // this CTA's blocks with a larger / an equal key
    __shared__ uint32_t s_prefix;
    __shared__ int s_remaining, s_take;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int r = blockIdx.x / SC_CTAS, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t below = (1u << lane) - 1u;
    const int n_keys = base_pos + r + 1, n_blocks = n_keys / ratio;
    const float *sc = scores + (size_t)r * max_blocks;
    uint8_t *m = mask + (size_t)r * max_ctx;
    uint32_t *l = list + (size_t)r * list_stride;
    const int tail0 = n_blocks * ratio;
    const int lo = min(rank * per_cta, n_blocks), hi = min(lo + per_cta, n_blocks);

    // this CTA's share of the mask, [m_lo, m_hi): 0 over the blocks, 1 over the tail; 16 bytes per
    // store where the addresses allow (shares are cut at multiples of 16 bytes of the row's address)
    {
        const uintptr_t a0 = (uintptr_t)m;
        const int64_t span = ((int64_t)n_keys + SC_CTAS - 1) / SC_CTAS;
        int64_t c0 = (int64_t)rank * span, c1 = c0 + span;
        c0 = rank == 0 ? 0 : (int64_t)(((a0 + c0 + 15) & ~(uintptr_t)15) - a0);
        c1 = rank == SC_CTAS - 1 ? n_keys : (int64_t)(((a0 + c1 + 15) & ~(uintptr_t)15) - a0);
        const int m_lo = (int)(c0 < n_keys ? c0 : n_keys), m_hi = (int)(c1 < n_keys ? c1 : n_keys);
        const int head = min(m_lo + (int)((16 - ((a0 + m_lo) & 15)) & 15), m_hi);
        const int zero_end = min(m_hi, tail0);
        const int vec_end = zero_end > head ? head + ((zero_end - head) & ~15) : head;
        for (int t = m_lo + tid; t < head; t += SC_THREADS) m[t] = t >= tail0;
        for (int t = head + 16 * tid; t < vec_end; t += 16 * SC_THREADS) *reinterpret_cast<uint4 *>(m + t) = make_uint4(0, 0, 0, 0);
        for (int t = vec_end + tid; t < m_hi; t += SC_THREADS) m[t] = t >= tail0;
    }
    // the scores of this CTA's blocks, once, as keys
    for (int i = tid; i < per_cta; i += SC_THREADS) {
        uint32_t key = 0;
        const int b = lo + i;
        if (b < hi) { uint32_t k2; if (sel_key(sc[b], k2)) key = k2; }
        keys[i] = key;
    }
    if (tid == 0) { s_prefix = 0; s_remaining = 0; s_take = 0; }
    __syncthreads();

    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix, high = shift == 24 ? 0u : 0xFFFFFFFFu << (shift + 8);
        for (int i = tid; i < per_cta; i += SC_THREADS) {        // the same trip count on every lane
            const uint32_t key = keys[i];
            const bool in = key != 0u && (key & high) == prefix;
            const int bin = in ? (int)((key >> shift) & 0xFF) : -1;
            // lanes of one bin add once: scores of a row mostly share their top bytes
            const uint32_t same = __match_any_sync(0xffffffffu, bin);
            if (in && (same & below) == 0u) atomicAdd(&hist[bin], __popc(same));
        }
        cluster.sync();                                           // every CTA's histogram is complete
        if (tid < 256) {
            int sum = 0;
#pragma unroll
            for (int q = 0; q < SC_CTAS; q++) sum += cluster.map_shared_rank(hist, q)[tid];
            tot[tid] = sum;
        }
        __syncthreads();
        // as in qsa_select_kernel: walking down from bin 255, the first bin at which the count reaches
        // `want` holds the key looked for (every CTA computes the same)
        if (warp == 0) {
            int want = s_remaining;
            __syncwarp();
            int h[8], mine = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) { h[j] = tot[255 - 8 * lane - j]; mine += h[j]; }
            int incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const int all = __shfl_sync(0xffffffffu, incl, 31);
            if (shift == 24) {
                want = min(min(block_topk, n_blocks), all);
                if (lane == 0) s_take = want;
            }
            const uint32_t reached = __ballot_sync(0xffffffffu, incl >= want);
            if (reached == 0u) {
                if (lane == 31) { s_remaining = want - (all - h[7]); s_prefix = prefix; }
            } else if (lane == __ffs(reached) - 1) {
                int run = incl - mine, bin = 0, rem = 0;
                bool done = false;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (!done && (run + h[j] >= want || 8 * lane + j == 255)) { bin = 255 - 8 * lane - j; rem = want - run; done = true; }
                    run += h[j];
                }
                s_remaining = rem;
                s_prefix = prefix | ((uint32_t)bin << shift);
            }
        }
        cluster.sync();                                           // all have read the histograms; the decision is visible
        if (s_take <= 0) break;                                   // (the same on every CTA)
    }
    const int take = s_take;
    const uint32_t kth = s_prefix;
    const int need_eq = s_remaining;

    // this warp's stretch of this CTA's keys (per_cta is a multiple of 1024, so a multiple of 32 per warp)
    const int chunk = per_cta / SC_WARPS;
    const int w_lo = warp * chunk, w_hi = w_lo + chunk;
    int gt = 0, eq = 0;
    if (take > 0)
        for (int i = w_lo + lane; i < w_hi; i += 32) {
            const uint32_t key = keys[i];
            gt += key != 0u && key > kth; eq += key != 0u && key == kth;
        }
    gt = (int)__reduce_add_sync(0xffffffffu, (unsigned)gt);
    eq = (int)__reduce_add_sync(0xffffffffu, (unsigned)eq);
    if (lane == 0) { w_gt[warp] = gt; w_eq[warp] = eq; }
    __syncthreads();
    if (tid == 0) {
        int g = 0, e = 0;
        for (int w = 0; w < SC_WARPS; w++) { g += w_gt[w]; e += w_eq[w]; }
        cta_cnt[0] = g; cta_cnt[1] = e;
    }
    cluster.sync();
    // equals and taken blocks in the CTAs before this one, then in the warps before this one
    int eq_before = 0, out_before = 0, total_taken = 0;
    {
        int e_run = 0, o_run = 0;
        for (int q = 0; q < SC_CTAS; q++) {
            const int *cnt = cluster.map_shared_rank(cta_cnt, q);
            const int g = cnt[0], e = cnt[1];
            if (q == rank) { eq_before = e_run; out_before = o_run; }
            o_run += g + min(max(need_eq - e_run, 0), e);
            e_run += e;
        }
        total_taken = o_run;
    }
    int eq_rank = eq_before, at = out_before;
    for (int w = 0; w < warp; w++) {
        at += w_gt[w] + min(max(need_eq - eq_rank, 0), w_eq[w]);
        eq_rank += w_eq[w];
    }
    if (take > 0) {
        for (int i = w_lo + lane; i < w_hi; i += 32) {
            const uint32_t key = keys[i];
            const int b = lo + i;
            const bool is_gt = key != 0u && key > kth, is_eq = key != 0u && key == kth;
            const uint32_t eq_bits = __ballot_sync(0xffffffffu, is_eq);
            const bool taken = is_gt || (is_eq && eq_rank + __popc(eq_bits & below) < need_eq);
            const uint32_t t_bits = __ballot_sync(0xffffffffu, taken);
            if (taken) {
                const int pos = (at + __popc(t_bits & below)) * ratio;
                for (int t = 0; t < ratio; t++) {
                    m[b * ratio + t] = 1;
                    l[1 + pos + t] = (uint32_t)(b * ratio + t);
                }
            }
            eq_rank += __popc(eq_bits);
            at += __popc(t_bits);
        }
    }
    if (rank == 0) {
        const int total = total_taken * ratio;
        for (int t = tail0 + tid; t < n_keys; t += SC_THREADS) l[1 + total + (t - tail0)] = (uint32_t)t;
        if (tid == 0) l[0] = (uint32_t)(total + (n_keys - tail0));
    }
    cluster.sync();                                               // no CTA leaves while another may still read its counts
}

}  // namespace

void launch_qsa_pool(cudaStream_t s, float *pool, const float *ikeys, const uint16_t *k_norm, const float *inv_freq, int d, int ratio,
                     int b0, int b1, float eps) {
    if (b1 <= b0) return;
    qsa_pool_kernel<<<(b1 - b0 + 7) / 8, 256, 0, s>>>(pool, ikeys, k_norm, inv_freq, d, ratio, b0, b1, eps);
    g_launches++;
}
void launch_qsa_scores(cudaStream_t s, float *scores, const float *qn, const float *pool, int rows, int nq, int d, int ratio,
                       int base_pos, int max_blocks) {
    const int most = std::min((base_pos + rows) / ratio, max_blocks);
    if (most <= 0 || rows <= 0) return;
    qsa_scores_kernel<<<dim3((most + 7) / 8, rows), 256, 0, s>>>(scores, qn, pool, nq, d, ratio, base_pos, max_blocks);
    g_launches++;
}
void launch_qsa_select(cudaStream_t s, uint8_t *mask, uint32_t *list, const float *scores, int rows, int ratio, int base_pos,
                       int block_topk, int max_ctx, int max_blocks) {
    if (rows <= 0) return;
    // long rows: a cluster of eight CTAs per row with the row's keys resident in their shared memory
    const int most = std::min((base_pos + rows) / ratio, max_blocks);
    const int per_cta = ((most + SC_CTAS - 1) / SC_CTAS + 1023) / 1024 * 1024;
    if (most >= 8192 && per_cta * 4 <= 200 * 1024) {
        static bool configured[64] = {false};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            cudaFuncSetAttribute(qsa_select_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            configured[dev] = true;
        }
        qsa_select_cluster_kernel<<<rows * SC_CTAS, SC_THREADS, (size_t)per_cta * 4, s>>>(mask, list, scores, ratio, base_pos, block_topk,
                                                                                         max_ctx, max_blocks, 1 + block_topk * ratio + ratio,
                                                                                         per_cta);
        g_launches++;
        return;
    }
    qsa_select_kernel<<<rows, SEL_THREADS, 0, s>>>(mask, list, scores, ratio, base_pos, block_topk, max_ctx, max_blocks,
                                                      1 + block_topk * ratio + ratio);
    g_launches++;
}

}  // namespace qw
