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

// One CTA per row.  taken[]: one bit per complete block, in dynamic shared memory.
constexpr int SEL_THREADS = 256;
__global__ void __launch_bounds__(SEL_THREADS) qsa_select_kernel(uint8_t *__restrict__ mask, uint32_t *__restrict__ list,
                                                                 const float *__restrict__ scores, int ratio, int base_pos,
                                                                 int block_topk, int max_ctx, int max_blocks, int list_stride) {
    extern __shared__ uint32_t taken[];
    __shared__ float red_v[SEL_THREADS / 32];
    __shared__ int red_i[SEL_THREADS / 32];
    __shared__ int chosen;
    __shared__ int counts[SEL_THREADS];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_keys = base_pos + r + 1, n_blocks = n_keys / ratio;
    const float *sc = scores + (size_t)r * max_blocks;
    uint8_t *m = mask + (size_t)r * max_ctx;
    uint32_t *l = list + (size_t)r * list_stride;
    for (int t = tid; t < n_keys; t += SEL_THREADS) m[t] = t >= n_blocks * ratio;
    for (int w = tid; w < (n_blocks + 31) / 32; w += SEL_THREADS) taken[w] = 0;
    __syncthreads();
    const int take = min(block_topk, n_blocks);
    for (int n = 0; n < take; n++) {
        // the best block not yet taken: the largest score above -FLT_MAX, the lowest index among equals
        float bv = 0.0f;
        int bi = -1;
        for (int b = tid; b < n_blocks; b += SEL_THREADS) {
            if ((taken[b >> 5] >> (b & 31)) & 1u) continue;
            const float v = sc[b];
            if (v > -FLT_MAX && (bi < 0 || v > bv)) { bv = v; bi = b; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if (lane == 0) { red_v[warp] = bv; red_i[warp] = bi; }
        __syncthreads();
        if (tid == 0) {
            float v = red_v[0];
            int i = red_i[0];
            for (int w = 1; w < SEL_THREADS / 32; w++)
                if (red_i[w] >= 0 && (i < 0 || red_v[w] > v || (red_v[w] == v && red_i[w] < i))) { v = red_v[w]; i = red_i[w]; }
            chosen = i;
            if (i >= 0) taken[i >> 5] |= 1u << (i & 31);
        }
        __syncthreads();
        if (chosen < 0) break;                                    // nothing above -FLT_MAX is left (block-uniform)
    }
    // mask of the taken blocks, and the list: taken blocks in ascending order, then the tail
    const int per = (n_blocks + SEL_THREADS - 1) / SEL_THREADS;
    const int lo = min(tid * per, n_blocks), hi = min(lo + per, n_blocks);
    int cnt = 0;
    for (int b = lo; b < hi; b++) cnt += (taken[b >> 5] >> (b & 31)) & 1u;
    counts[tid] = cnt;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int i = 0; i < SEL_THREADS; i++) { const int c2 = counts[i]; counts[i] = run; run += c2; }
        chosen = run;                                             // blocks taken in all
    }
    __syncthreads();
    int at = counts[tid] * ratio;
    for (int b = lo; b < hi; b++) {
        if (!((taken[b >> 5] >> (b & 31)) & 1u)) continue;
        for (int t = 0; t < ratio; t++) {
            m[b * ratio + t] = 1;
            l[1 + at++] = (uint32_t)(b * ratio + t);
        }
    }
    const int tail0 = n_blocks * ratio, total = chosen * ratio;
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
    const size_t smem = (size_t)((max_blocks + 31) / 32 + 1) * sizeof(uint32_t);
    qsa_select_kernel<<<rows, SEL_THREADS, smem, s>>>(mask, list, scores, ratio, base_pos, block_topk, max_ctx, max_blocks,
                                                      1 + block_topk * ratio + ratio);
    g_launches++;
}

}  // namespace qw
