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
    pdl_wait();                                                   // the index keys may come from the kernel before
    pdl_launch_next();
    if (b >= b1) return;
    float x[8];
    block_key(x, ikeys, k_norm, inv_freq, d, ratio, b, eps, lane);
#pragma unroll
    for (int k = 0; k < 8; k++)
        if (k < (d >> 5)) pool[(size_t)b * d + lane + 32 * k] = x[k];
}

// Scores, a LANE per block key.  A warp takes 32 consecutive block keys: their d floats travel into shared
// memory with 16-byte asynchronous copies, 32 dims at a time in two stages (rows padded by 4 floats, so a
// lane reading its own row 16 bytes at a time meets no bank conflict), and each lane then walks its key
// once with one multiply-add chain per index head, the queries read from shared memory as broadcasts.
// About 25 instructions per key instead of 320: the kernel with a warp per key reloaded the queries and
// ran a five-step shuffle sum for every (key, head), and sat at 88 % issue utilisation at 1.3 TB/s.
// Used when d is a multiple of 32; the sums run over d in index order in both scoring ops, so scores from
// stored block keys still equal scores from raw keys bit for bit.
constexpr int SCL_WARPS = 4, SCL_CH = 32, SCL_LD = SCL_CH + 4, SCL_HB = 4, SCL_PIECES = SCL_CH / 4;
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *src, bool valid) {
    const int n = valid ? 16 : 0;                                 // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(src), "r"(n) : "memory");
}
__global__ void __launch_bounds__(SCL_WARPS * 32) qsa_scores_lane_kernel(float *__restrict__ scores, const float *__restrict__ qn,
                                                                         const float *__restrict__ pool, int nq, int d, int ratio,
                                                                         int base_pos, int max_blocks) {
    extern __shared__ __align__(16) float scl_smem[];             // [nq][d] queries | per warp [2 stages][32 keys][SCL_LD]
    const int r = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_blocks = min((base_pos + r + 1) / ratio, max_blocks);
    const int b0 = (blockIdx.x * SCL_WARPS + warp) * 32;
    float *qs = scl_smem, *ks = scl_smem + nq * d + (size_t)warp * 2 * 32 * SCL_LD;
    pdl_wait();                                                   // the queries and the pool may come from the kernel before
    pdl_launch_next();
    for (int i = threadIdx.x * 4; i < nq * d; i += SCL_WARPS * 32 * 4)
        *reinterpret_cast<float4 *>(qs + i) = __ldg(reinterpret_cast<const float4 *>(qn + (size_t)r * nq * d + i));
    const int n_ch = d / SCL_CH;
    // step t of the walk = (pass over four index heads, chunk of SCL_CH dims): chunk t % n_ch into stage t & 1; the
    // lanes share out the 16-byte pieces of the warp's 32 rows
    const int passes = (nq + SCL_HB - 1) / SCL_HB, steps = passes * n_ch;
    auto stage = [&](int t) {
        float *dst = ks + (size_t)(t & 1) * 32 * SCL_LD;
        const int c = t % n_ch;
#pragma unroll
        for (int i = lane; i < 32 * SCL_PIECES; i += 32) {
            const int row = i / SCL_PIECES, piece = i % SCL_PIECES, b = b0 + row;
            cp_async16(dst + row * SCL_LD + piece * 4, pool + (size_t)min(b, max_blocks - 1) * d + c * SCL_CH + piece * 4, b < n_blocks);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (b0 < n_blocks) stage(0);
    __syncthreads();                                              // the queries are in place
    if (b0 >= n_blocks) return;
    float total = 0.0f;
    float acc[SCL_HB] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int t = 0; t < steps; t++) {
        const int c = t % n_ch, h0 = (t / n_ch) * SCL_HB;
        if (t + 1 < steps) { stage(t + 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        const float *krow = ks + (size_t)(t & 1) * 32 * SCL_LD + lane * SCL_LD;
        const float *q = qs + (size_t)h0 * d + c * SCL_CH;
#pragma unroll 4
        for (int j = 0; j < SCL_CH; j += 4) {
            const float4 k4 = *reinterpret_cast<const float4 *>(krow + j);
#pragma unroll
            for (int h = 0; h < SCL_HB; h++) {
                if (h0 + h < nq) {
                    const float4 q4 = *reinterpret_cast<const float4 *>(q + (size_t)h * d + j);
                    acc[h] = fmaf(k4.w, q4.w, fmaf(k4.z, q4.z, fmaf(k4.y, q4.y, fmaf(k4.x, q4.x, acc[h]))));
                }
            }
        }
        __syncwarp();                                             // the stage may be written again
        if (c == n_ch - 1) {                                      // a pass is complete: its heads join the sum
#pragma unroll
            for (int h = 0; h < SCL_HB; h++) {
                if (h0 + h < nq && acc[h] > 0.0f) total = __fadd_rn(total, acc[h]);
                acc[h] = 0.0f;
            }
        }
    }
    const int b = b0 + lane;
    if (b < n_blocks) scores[(size_t)r * max_blocks + b] = __fdiv_rn(total, sqrtf((float)d));
}

// one warp per (row, block): grid (ceil(max visible blocks / 8), rows)
__global__ void __launch_bounds__(256) qsa_scores_kernel(float *__restrict__ scores, const float *__restrict__ qn,
                                                         const float *__restrict__ pool, int nq, int d, int ratio, int base_pos,
                                                         int max_blocks) {
    const int r = blockIdx.y, b = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int n_blocks = (base_pos + r + 1) / ratio;
    pdl_wait();
    pdl_launch_next();
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

// One CTA per row.  The reference's CPU statement finds the block_topk best blocks one at a time (the
// largest score above -FLT_MAX, the lowest index among equals, qwasar_flash_cpu.c:345-418); its GPU
// kernel is qw_qsa_select, metal/sparse.metal:958-1049.  Both pick the first `take` blocks in the order
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
    pdl_wait();                                                   // (the kernel before may still read the mask and the list)
    pdl_launch_next();
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
// (0 = not selectable), and every later pass runs from there.  Three radix passes (11, 11 and 10 bits)
// each build a histogram per CTA (warp-aggregated adds) in a buffer of their own, so the cluster
// synchronises ONCE per pass: every CTA then sums the eight histograms through distributed shared
// memory and takes the same decision with a block-wide scan from the top bin down.  (Four 8-bit
// passes with two cluster barriers each took 26 us on 65 536 scores, nearly all of it waiting at
// barriers.)  The ordered passes need only each CTA's counts of larger and equal keys, read the same
// way.  The mask is cleared and the list written by the CTAs in parallel, each for its own stretch.
namespace cg = cooperative_groups;
constexpr int SC_CTAS = 8, SC_THREADS = 1024, SC_WARPS = SC_THREADS / 32, SC_BINS = 2048, SC_REP = 2, SC_PRE = 8;
static_assert(SC_BINS == 2 * SC_THREADS, "the scan gives every thread two bins");

__global__ void __cluster_dims__(SC_CTAS, 1, 1) __launch_bounds__(SC_THREADS)
qsa_select_cluster_kernel(uint8_t *__restrict__ mask, uint32_t *__restrict__ list, const float *__restrict__ scores, int ratio,
                          int base_pos, int block_topk, int max_ctx, int max_blocks, int list_stride, int per_cta) {
    extern __shared__ uint32_t keys[];                            // per_cta keys of this CTA's blocks
    int (*hist)[SC_BINS] = reinterpret_cast<int (*)[SC_BINS]>(keys + per_cta);     // one histogram per pass (dynamic, behind the keys)
    int (*rep0)[SC_BINS] = hist + 3;                              // pass 0 counts into SC_REP copies (hist[0] is the first)
    __shared__ int tot[SC_BINS];
    __shared__ int w_sum[SC_WARPS], w_off[SC_WARPS], s_all;
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

    // under the kernel before (programmatic dependent launch): the histograms are cleared; then it has completed
    for (int i = tid; i < 3 * SC_BINS; i += SC_THREADS) (&hist[0][0])[i] = 0;
    for (int i = tid; i < (SC_REP - 1) * SC_BINS; i += SC_THREADS) (&rep0[0][0])[i] = 0;
    if (tid == 0) { s_prefix = 0; s_remaining = 0; s_take = 0; }
    pdl_wait();
    pdl_launch_next();
    // the scores of this CTA's blocks are asked for first (up to SC_PRE per thread stay in registers), so that their
    // trip to memory runs under the clearing of the mask
    float pre[SC_PRE];
#pragma unroll
    for (int j = 0; j < SC_PRE; j++) {
        const int b = lo + tid + j * SC_THREADS;
        pre[j] = b < hi ? sc[b] : -FLT_MAX;
    }
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
    // ... and go to shared memory as keys
#pragma unroll
    for (int j = 0; j < SC_PRE; j++) {
        const int i = tid + j * SC_THREADS;
        uint32_t key = 0, k2;
        if (i < per_cta) { if (sel_key(pre[j], k2)) key = k2; keys[i] = key; }
    }
    for (int i = tid + SC_PRE * SC_THREADS; i < per_cta; i += SC_THREADS) {
        uint32_t key = 0;
        const int b = lo + i;
        if (b < hi) { uint32_t k2; if (sel_key(sc[b], k2)) key = k2; }
        keys[i] = key;
    }
    __syncthreads();

    for (int pass = 0; pass < 3; pass++) {
        const int shift = pass == 0 ? 21 : pass == 1 ? 10 : 0, nbits = pass == 2 ? 10 : 11;
        const uint32_t prefix = s_prefix, high = pass == 0 ? 0u : 0xFFFFFFFFu << (shift + nbits), bmask = (1u << nbits) - 1u;
        int want = s_remaining;                                   // (read before this pass's decision is written)
        // The first pass sees every key, and the top bits of a row's scores take a handful of values: its adds go to
        // one of SC_REP copies by warp, folded into one histogram before the cluster looks at it (two copies measured
        // best: 20.3 us for the whole selection against 21.7 with eight, whose clearing and folding cost more than
        // they save).
        int *h = pass == 0 && (warp % SC_REP) ? rep0[warp % SC_REP - 1] : hist[pass];
        // One add per key, no aggregation inside the warp: matching the lanes' bins first (match.any) costs a round per
        // distinct value, and with a few dozen distinct bins per warp that was 4 of the first pass's 5 us; electing the
        // two most common bins of a warp was slower too (24.5 against 21 us), and rows of equal scores (all zero, nine in
        // ten zero) cost plain adds nothing extra: the hardware folds a warp's adds to one address.  The later passes only
        // add the few keys that share the prefix.
        for (int i = tid; i < per_cta; i += SC_THREADS) {
            const uint32_t key = keys[i];
            if (key != 0u && (key & high) == prefix) atomicAdd(&h[(key >> shift) & bmask], 1);
        }
        if (pass == 0) {
            __syncthreads();
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int bin = tid + j * SC_THREADS;
                int sum = hist[0][bin];
#pragma unroll
                for (int q = 0; q < SC_REP - 1; q++) sum += rep0[q][bin];
                hist[0][bin] = sum;
            }
        }
        cluster.sync();                                           // every CTA's histogram of this pass is complete
        // CTA q adds up its eighth of the bins over the eight CTAs and stores the sums into every CTA's `tot`
        // (each CTA pulling all eight histograms moved four times the bytes between the SMs and took 2 us a pass)
        {
            const int bins = 1 << nbits, per = bins / SC_CTAS;
            if (tid < per) {
                const int bin = rank * per + tid;
                int v[SC_CTAS];
#pragma unroll
                for (int q = 0; q < SC_CTAS; q++) v[q] = cluster.map_shared_rank(hist[pass], q)[bin];
                int sum = 0;
#pragma unroll
                for (int q = 0; q < SC_CTAS; q++) sum += v[q];
#pragma unroll
                for (int q = 0; q < SC_CTAS; q++) cluster.map_shared_rank(tot, q)[bin] = sum;
            }
            if (bins < SC_BINS) for (int bin = bins + tid; bin < SC_BINS; bin += SC_THREADS) tot[bin] = 0;
        }
        cluster.sync();                                           // every CTA's `tot` is complete
        // From the top bin down, the first bin at which the running count reaches `want` holds the key looked
        // for; every CTA computes the same.  Thread t owns bins B - 1 - 2t and B - 2 - 2t.
        const int bhi = SC_BINS - 1 - 2 * tid;
        const int c0 = tot[bhi], c1 = tot[bhi - 1], mine = c0 + c1;
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) w_sum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const int v = w_sum[lane];
            int iv = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, iv, o);
                if (lane >= o) iv += up;
            }
            w_off[lane] = iv - v;
            if (lane == 31) s_all = iv;
        }
        __syncthreads();
        incl += w_off[warp];
        const int excl = incl - mine, all = s_all;
        if (pass == 0) {
            want = min(min(block_topk, n_blocks), all);
            if (tid == 0) s_take = want;
        }
        if (want > 0) {
            if (excl < want && want <= incl) {
                const bool first = excl + c0 >= want;
                s_prefix = prefix | ((uint32_t)(first ? bhi : bhi - 1) << shift);
                s_remaining = first ? want - excl : want - excl - c0;
            } else if (all < want && tid == SC_THREADS - 1) {     // (cannot happen: the prefix bin held at least `want`)
                s_prefix = prefix;
                s_remaining = want - (all - c1);
            }
        }
        __syncthreads();                                          // the decision is visible
        if (want <= 0) break;                                     // (the same on every CTA)
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
        int gq[SC_CTAS], eq_q[SC_CTAS];
#pragma unroll
        for (int q = 0; q < SC_CTAS; q++) {                       // (all the remote reads in flight together)
            const int *cnt = cluster.map_shared_rank(cta_cnt, q);
            gq[q] = cnt[0]; eq_q[q] = cnt[1];
        }
#pragma unroll
        for (int q = 0; q < SC_CTAS; q++) {
            const int g = gq[q], e = eq_q[q];
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
                if (ratio == 4 && (((uintptr_t)m) & 3) == 0) {    // the usual block of four tokens: one store for its mask bytes
                    *reinterpret_cast<uint32_t *>(m + b * 4) = 0x01010101u;
                    const uint32_t p0 = (uint32_t)(b * 4);
                    l[1 + pos] = p0; l[2 + pos] = p0 + 1; l[3 + pos] = p0 + 2; l[4 + pos] = p0 + 3;
                } else {
                    for (int t = 0; t < ratio; t++) {
                        m[b * ratio + t] = 1;
                        l[1 + pos + t] = (uint32_t)(b * ratio + t);
                    }
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

// The launch may start under the kernel in front of it on the stream; the kernel orders itself with pdl_wait().
static void pdl_attr(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr, cudaStream_t s) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_tune_pdl ? 1 : 0; cfg.stream = s;
}

void launch_qsa_pool(cudaStream_t s, float *pool, const float *ikeys, const uint16_t *k_norm, const float *inv_freq, int d, int ratio,
                     int b0, int b1, float eps) {
    if (b1 <= b0) return;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    pdl_attr(cfg, attr, s);
    cfg.gridDim = dim3((b1 - b0 + 7) / 8); cfg.blockDim = dim3(256);
    if (cudaLaunchKernelEx(&cfg, qsa_pool_kernel, pool, ikeys, k_norm, inv_freq, d, ratio, b0, b1, eps) == cudaSuccess) g_launches++;
}
void launch_qsa_scores(cudaStream_t s, float *scores, const float *qn, const float *pool, int rows, int nq, int d, int ratio,
                       int base_pos, int max_blocks) {
    const int most = std::min((base_pos + rows) / ratio, max_blocks);
    if (most <= 0 || rows <= 0) return;
    const size_t smem = ((size_t)nq * d + (size_t)SCL_WARPS * 2 * 32 * SCL_LD) * sizeof(float);
    if (d % SCL_CH == 0 && ((reinterpret_cast<uintptr_t>(pool) | reinterpret_cast<uintptr_t>(qn)) & 15) == 0 && smem <= 200 * 1024) {
        static bool configured[16] = {false};
        int dev = 0; cudaGetDevice(&dev);
        if (dev >= 0 && dev < 16 && !configured[dev]) {
            cudaFuncSetAttribute(qsa_scores_lane_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            configured[dev] = true;
        }
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        pdl_attr(cfg, attr, s);
        cfg.gridDim = dim3((most + SCL_WARPS * 32 - 1) / (SCL_WARPS * 32), rows); cfg.blockDim = dim3(SCL_WARPS * 32); cfg.dynamicSmemBytes = smem;
        if (cudaLaunchKernelEx(&cfg, qsa_scores_lane_kernel, scores, qn, pool, nq, d, ratio, base_pos, max_blocks) == cudaSuccess) g_launches++;
        return;
    }
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    pdl_attr(cfg, attr, s);
    cfg.gridDim = dim3((most + 7) / 8, rows); cfg.blockDim = dim3(256);
    if (cudaLaunchKernelEx(&cfg, qsa_scores_kernel, scores, qn, pool, nq, d, ratio, base_pos, max_blocks) == cudaSuccess) g_launches++;
}
void launch_qsa_select(cudaStream_t s, uint8_t *mask, uint32_t *list, const float *scores, int rows, int ratio, int base_pos,
                       int block_topk, int max_ctx, int max_blocks) {
    if (rows <= 0) return;
    // long rows: a cluster of eight CTAs per row with the row's keys resident in their shared memory
    const int most = std::min((base_pos + rows) / ratio, max_blocks);
    const int per_cta = ((most + SC_CTAS - 1) / SC_CTAS + 1023) / 1024 * 1024;
    if (most >= 8192 && per_cta * 4 <= 120 * 1024) {
        static bool configured[64] = {false};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            cudaFuncSetAttribute(qsa_select_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
            configured[dev] = true;
        }
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        pdl_attr(cfg, attr, s);
        cfg.gridDim = dim3(rows * SC_CTAS); cfg.blockDim = dim3(SC_THREADS); cfg.dynamicSmemBytes = (size_t)per_cta * 4 + (size_t)(3 + SC_REP - 1) * SC_BINS * 4;
        if (cudaLaunchKernelEx(&cfg, qsa_select_cluster_kernel, mask, list, scores, ratio, base_pos, block_topk, max_ctx, max_blocks,
                               1 + block_topk * ratio + ratio, per_cta) == cudaSuccess) g_launches++;
        return;
    }
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    pdl_attr(cfg, attr, s);
    cfg.gridDim = dim3(rows); cfg.blockDim = dim3(SEL_THREADS);
    if (cudaLaunchKernelEx(&cfg, qsa_select_kernel, mask, list, scores, ratio, base_pos, block_topk, max_ctx, max_blocks,
                           1 + block_topk * ratio + ratio) == cudaSuccess) g_launches++;
}

}  // namespace qw
