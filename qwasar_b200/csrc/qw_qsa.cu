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
// pass is one sweep over the row's scores, each thread over a contiguous run of blocks, which is
// also what orders the equals and the list.
constexpr int SEL_THREADS = 256;
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
    __shared__ int counts[SEL_THREADS];
    __shared__ uint32_t s_prefix;
    __shared__ int s_remaining, s_total;
    const int r = blockIdx.x, tid = threadIdx.x;
    const int n_keys = base_pos + r + 1, n_blocks = n_keys / ratio;
    const float *sc = scores + (size_t)r * max_blocks;
    uint8_t *m = mask + (size_t)r * max_ctx;
    uint32_t *l = list + (size_t)r * list_stride;
    const int per = (n_blocks + SEL_THREADS - 1) / SEL_THREADS;
    const int lo = min(tid * per, n_blocks), hi = min(lo + per, n_blocks);
    for (int t = tid; t < n_keys; t += SEL_THREADS) m[t] = t >= n_blocks * ratio;

    // how many blocks can be selected at all
    int eligible = 0;
    for (int b = lo; b < hi; b++) { uint32_t key; eligible += sel_key(sc[b], key); }
    counts[tid] = eligible;
    __syncthreads();
    if (tid == 0) {
        int e = 0;
        for (int i = 0; i < SEL_THREADS; i++) e += counts[i];
        s_remaining = min(min(block_topk, n_blocks), e);          // take
        s_prefix = 0;
    }
    __syncthreads();
    const int take = s_remaining;

    // radix select: after the pass over byte `shift`, s_prefix holds the top bytes of the key of
    // the take-th best block and s_remaining how many blocks with that prefix are still wanted
    if (take > 0) {
        for (int shift = 24; shift >= 0; shift -= 8) {
            hist[tid] = 0;                                        // SEL_THREADS == 256 bins
            __syncthreads();
            const uint32_t prefix = s_prefix, high = shift == 24 ? 0u : 0xFFFFFFFFu << (shift + 8);
            for (int b = lo; b < hi; b++) {
                uint32_t key;
                if (sel_key(sc[b], key) && (key & high) == prefix) atomicAdd(&hist[(key >> shift) & 0xFF], 1);
            }
            __syncthreads();
            if (tid == 0) {
                int want = s_remaining, bin = 255;
                for (; bin > 0 && hist[bin] < want; bin--) want -= hist[bin];
                s_remaining = want;                               // still wanted among the keys of this bin
                s_prefix = prefix | ((uint32_t)bin << shift);
            }
            __syncthreads();
        }
    }
    const uint32_t kth = s_prefix;                                // the key of the take-th best block
    const int need_eq = s_remaining;                              // blocks with exactly that key to take, lowest index first

    // equals before this thread's run, then the verdict per block; taken blocks counted for the list
    int eq = 0;
    if (take > 0)
        for (int b = lo; b < hi; b++) { uint32_t key; eq += sel_key(sc[b], key) && key == kth; }
    counts[tid] = eq;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int i = 0; i < SEL_THREADS; i++) { const int c2 = counts[i]; counts[i] = run; run += c2; }
    }
    __syncthreads();
    const int eq_base = counts[tid];
    __syncthreads();
    int cnt = 0;
    if (take > 0) {
        int rank = eq_base;
        for (int b = lo; b < hi; b++) {
            uint32_t key;
            if (sel_key(sc[b], key)) cnt += key > kth || (key == kth && rank++ < need_eq);
        }
    }
    counts[tid] = cnt;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int i = 0; i < SEL_THREADS; i++) { const int c2 = counts[i]; counts[i] = run; run += c2; }
        s_total = run;                                            // blocks taken in all (== take)
    }
    __syncthreads();
    // the mask of the taken blocks, and the list: taken blocks in ascending order, then the tail
    if (take > 0) {
        int at = counts[tid] * ratio, rank = eq_base;
        for (int b = lo; b < hi; b++) {
            uint32_t key;
            if (!sel_key(sc[b], key)) continue;
            if (!(key > kth || (key == kth && rank++ < need_eq))) continue;
            for (int t = 0; t < ratio; t++) {
                m[b * ratio + t] = 1;
                l[1 + at++] = (uint32_t)(b * ratio + t);
            }
        }
    }
    const int tail0 = n_blocks * ratio, total = s_total * ratio;
    for (int t = tail0 + tid; t < n_keys; t += SEL_THREADS) l[1 + total + (t - tail0)] = (uint32_t)t;
    if (tid == 0) l[0] = (uint32_t)(total + (n_keys - tail0));
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
    qsa_select_kernel<<<rows, SEL_THREADS, 0, s>>>(mask, list, scores, ratio, base_pos, block_topk, max_ctx, max_blocks,
                                                      1 + block_topk * ratio + ratio);
    g_launches++;
}

}  // namespace qw
