/* CPU oracle for the gated GQA full-attention node -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic the reference performs for this
 * path, written so that every floating-point operation happens in the same
 * order as in the reference's scalar twins (qwasar_cpu.c).  Only the tests,
 * the smoke check and the benchmark's cpu_baseline leg may link or load this
 * file; the product library never does.
 *
 * Parity status: PINNED.  The test-suite holds this file bit-for-bit against
 * (a) the reference's own qwasar_cpu.c compiled unmodified into oracle/_ref
 * (see oracle/Makefile) on seeded inputs, (b) the fixtures under
 * tests/golden/ which were produced by that compiled reference, and (c) the
 * known answers the reference's tests hold for the rope tables
 * (tests/test_ops.c:163-182).
 *
 * The 16-bit cache element type is chosen per call: ORC_BF16 is what this
 * build stores (the reference source compiled with -D__fp16=__bf16), ORC_F16
 * is what the reference ships (qwasar_gpu.h:395-400).
 *
 * Build without -ffast-math and with -ffp-contract=off so that sums are
 * strict IEEE in program order. */

#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORC_BF16 = 0, ORC_F16 = 1 };

/* ---- 16-bit element conversions ------------------------------------------ */

/* bfloat16 widening: the 16 bits are the top half of the float
 * (qwasar_cpu.c:15-19). */
static inline float orc_bf16_up(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, sizeof f);
    return f;
}

/* float -> bfloat16, round to nearest even; what `(__bf16)v` does when
 * qwasar_cpu.c:337-342 is compiled with -D__fp16=__bf16. */
static inline uint16_t orc_bf16_down(float f) {
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* IEEE half, as the shipped reference stores it (qwasar_cpu.c:330-342). */
static inline float orc_f16_up(uint16_t h) {
    _Float16 x;
    memcpy(&x, &h, sizeof x);
    return (float)x;
}
static inline uint16_t orc_f16_down(float f) {
    _Float16 x = (_Float16)f;
    uint16_t h;
    memcpy(&h, &x, sizeof h);
    return h;
}

float orc_cache_up(uint16_t h, int fmt) { return fmt == ORC_F16 ? orc_f16_up(h) : orc_bf16_up(h); }
uint16_t orc_cache_down(float f, int fmt) { return fmt == ORC_F16 ? orc_f16_down(f) : orc_bf16_down(f); }

void orc_cache_down_n(uint16_t *dst, const float *src, size_t n, int fmt) {
    for (size_t i = 0; i < n; i++) dst[i] = orc_cache_down(src[i], fmt);
}
void orc_cache_up_n(float *dst, const uint16_t *src, size_t n, int fmt) {
    for (size_t i = 0; i < n; i++) dst[i] = orc_cache_up(src[i], fmt);
}

/* ---- the pre-ops ---------------------------------------------------------- */

/* q_proj's output holds, per head, the query then the output gate
 * (qwasar_gpu.h:391-393; metal/act.metal:46-61).  A pure copy. */
void orc_split_heads2(float *a, float *b, const float *src,
                      int32_t rows, int32_t heads, int32_t dim) {
    for (size_t rh = 0; rh < (size_t)rows * heads; rh++) {
        memcpy(a + rh * dim, src + rh * 2 * dim, (size_t)dim * sizeof(float));
        memcpy(b + rh * dim, src + rh * 2 * dim + dim, (size_t)dim * sizeof(float));
    }
}

/* RMS norm of each row of an [rows, dim] array (qwasar_cpu.c:68-82): the sum
 * of squares is taken left to right, the reciprocal root is one divide after
 * one sqrtf, out_scale multiplies the reciprocal, and the bf16 weight (NULL =
 * none) multiplies last. */
void orc_rms_norm(float *y, const float *x, const uint16_t *w_bf16,
                  int32_t dim, int32_t rows, float eps, float out_scale) {
    for (int32_t r = 0; r < rows; r++) {
        const float *xi = x + (size_t)r * dim;
        float *yo = y + (size_t)r * dim;
        float acc = 0.0f;
        for (int32_t i = 0; i < dim; i++) acc += xi[i] * xi[i];
        const float inv = 1.0f / sqrtf(acc / (float)dim + eps) * out_scale;
        for (int32_t i = 0; i < dim; i++) {
            float t = xi[i] * inv;
            yo[i] = w_bf16 ? t * orc_bf16_up(w_bf16[i]) : t;
        }
    }
}

/* Interleaved-MRoPE tables (qwasar_cpu.c:284-302): frequency j belongs to the
 * time axis unless j = d (mod 3) and j < 3*section[d] for d in {1,2}. */
void orc_rope_tables(uint8_t *axis, float *inv_freq, int32_t rotary_dim,
                     float theta, const int32_t section[3]) {
    const int32_t nfreq = rotary_dim / 2;
    for (int32_t j = 0; j < nfreq; j++) {
        int a = 0;
        for (int d = 1; d <= 2; d++) {
            int32_t lim = section[d] * 3 < nfreq ? section[d] * 3 : nfreq;
            if (j % 3 == d && j < lim) a = d;
        }
        axis[j] = (uint8_t)a;
        inv_freq[j] = 1.0f / powf(theta, (float)(2 * j) / (float)rotary_dim);
    }
}

/* Half-split rotation of the first rotary_dim dims, in place
 * (qwasar_cpu.c:304-319): pair (j, j+rotary_dim/2) turns by
 * (float)pos[axis[j]][r] * inv_freq[j], cos/sin evaluated in fp32. */
void orc_rope_partial(float *x, const int32_t *pos, const uint8_t *axis,
                      const float *inv_freq, int32_t rows, int32_t heads,
                      int32_t head_dim, int32_t rotary_dim) {
    const int32_t nfreq = rotary_dim / 2;
    for (int32_t r = 0; r < rows; r++) {
        for (int32_t j = 0; j < nfreq; j++) {
            const float ang = (float)pos[(size_t)axis[j] * rows + r] * inv_freq[j];
            const float cs = cosf(ang), sn = sinf(ang);
            for (int32_t h = 0; h < heads; h++) {
                float *v = x + ((size_t)r * heads + h) * head_dim;
                const float lo = v[j], hi = v[j + nfreq];
                v[j]         = lo * cs - hi * sn;
                v[j + nfreq] = hi * cs + lo * sn;
            }
        }
    }
}

/* KV append (qwasar_cpu.c:344-355): one rounding to the cache type, slot
 * [head][base_pos + row][dim] of a head-major [kv_heads, max_ctx, head_dim]
 * array. */
void orc_kv_write(uint16_t *kc, uint16_t *vc, const float *k, const float *v,
                  int32_t rows, int32_t kv_heads, int32_t head_dim,
                  int32_t max_ctx, int32_t base_pos, int fmt) {
    for (int32_t h = 0; h < kv_heads; h++)
        for (int32_t r = 0; r < rows; r++) {
            const size_t from = ((size_t)r * kv_heads + h) * head_dim;
            const size_t to = ((size_t)h * max_ctx + base_pos + r) * head_dim;
            orc_cache_down_n(kc + to, k + from, (size_t)head_dim, fmt);
            orc_cache_down_n(vc + to, v + from, (size_t)head_dim, fmt);
        }
}

/* ---- attention ------------------------------------------------------------ */

/* One (row, query head) of qwasar_cpu.c:357-391: scores s_t = sum_i
 * (q_i*scale)*K[t][i] left to right, m = max (starting from -FLT_MAX),
 * e_t = expf(s_t - m), sum left to right, out_i = sum_t (e_t/sum)*V[t][i]
 * left to right over t.  `work` holds n floats. */
static void orc_attend_one(float *o, const float *q, const uint16_t *kh,
                           const uint16_t *vh, int32_t n, int32_t head_dim,
                           float scale, int fmt, float *work) {
    float top = -FLT_MAX;
    for (int32_t t = 0; t < n; t++) {
        const uint16_t *kr = kh + (size_t)t * head_dim;
        float dot = 0.0f;
        if (fmt == ORC_BF16)
            for (int32_t i = 0; i < head_dim; i++) dot += q[i] * scale * orc_bf16_up(kr[i]);
        else
            for (int32_t i = 0; i < head_dim; i++) dot += q[i] * scale * orc_f16_up(kr[i]);
        work[t] = dot;
        if (dot > top) top = dot;
    }
    float denom = 0.0f;
    for (int32_t t = 0; t < n; t++) {
        work[t] = expf(work[t] - top);
        denom += work[t];
    }
    for (int32_t i = 0; i < head_dim; i++) o[i] = 0.0f;
    for (int32_t t = 0; t < n; t++) {
        const uint16_t *vr = vh + (size_t)t * head_dim;
        const float w = work[t] / denom;
        if (fmt == ORC_BF16)
            for (int32_t i = 0; i < head_dim; i++) o[i] += w * orc_bf16_up(vr[i]);
        else
            for (int32_t i = 0; i < head_dim; i++) o[i] += w * orc_f16_up(vr[i]);
    }
}

/* Causal attention of `rows` queries over a head-major cache: row r of query
 * head h reads kv head h / (q_heads/kv_heads) at positions [0, base_pos + r]
 * (qwasar_cpu.c:357-391; qwasar_gpu.h:408-413).  threads > 1 spreads the
 * independent (row, head) pairs over OpenMP threads without changing any
 * pair's arithmetic. */
void orc_attn_decode(float *out, const float *q, const uint16_t *kc,
                     const uint16_t *vc, int32_t rows, int32_t q_heads,
                     int32_t kv_heads, int32_t head_dim, int32_t max_ctx,
                     int32_t base_pos, float scale, int fmt, int threads) {
    const int32_t group = q_heads / kv_heads;
    const int32_t pairs = rows * q_heads;
    (void)threads;
#ifdef _OPENMP
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
#endif
    {
        float *work = (float *)malloc((size_t)(base_pos + rows) * sizeof(float));
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 1)
#endif
        for (int32_t p = 0; p < pairs; p++) {
            const int32_t r = p / q_heads, h = p % q_heads;
            const size_t head_off = (size_t)(h / group) * max_ctx * head_dim;
            orc_attend_one(out + (size_t)p * head_dim, q + (size_t)p * head_dim,
                           kc + head_off, vc + head_off, base_pos + r + 1,
                           head_dim, scale, fmt, work);
        }
        free(work);
    }
}

/* Attention that sees only listed cache positions (the QSA mask as a list):
 * row r of query head h attends positions list[r][1 .. 1 + list[r][0]) of kv
 * head h / (q_heads/kv_heads), in list order; list rows are list_stride
 * uint32 apart (a count, then positions ascending, entries past the count
 * unspecified) -- qwasar_gpu.h:635-645.  The arithmetic is the reference's
 * masked softmax (qwasar_flash_cpu.c:447-478: scores of the allowed
 * positions, max, expf, sum, weighted V), which over a list is
 * orc_attend_one on the listed rows: the K and V rows are gathered into a
 * dense run and attended like a cache of that many positions. */
void orc_attn_masked(float *out, const float *q, const uint16_t *kc, const uint16_t *vc,
                     const uint32_t *list, int32_t list_stride, int32_t rows, int32_t q_heads,
                     int32_t kv_heads, int32_t head_dim, int32_t max_ctx, float scale, int fmt) {
    const int32_t gqa = q_heads / kv_heads;
    for (int32_t r = 0; r < rows; r++) {
        const uint32_t *l = list + (size_t)r * list_stride;
        const int32_t n = (int32_t)l[0];
        uint16_t *kd = (uint16_t *)malloc((size_t)(n ? n : 1) * head_dim * 2);
        uint16_t *vd = (uint16_t *)malloc((size_t)(n ? n : 1) * head_dim * 2);
        float *work = (float *)malloc((size_t)(n ? n : 1) * sizeof(float));
        for (int32_t kvh = 0; kvh < kv_heads; kvh++) {
            for (int32_t j = 0; j < n; j++) {
                memcpy(kd + (size_t)j * head_dim, kc + ((size_t)kvh * max_ctx + l[1 + j]) * head_dim, (size_t)head_dim * 2);
                memcpy(vd + (size_t)j * head_dim, vc + ((size_t)kvh * max_ctx + l[1 + j]) * head_dim, (size_t)head_dim * 2);
            }
            for (int32_t g = 0; g < gqa; g++) {
                const size_t p = (size_t)r * q_heads + (size_t)kvh * gqa + g;
                if (n > 0) orc_attend_one(out + p * head_dim, q + p * head_dim, kd, vd, n, head_dim, scale, fmt, work);
                else memset(out + p * head_dim, 0, (size_t)head_dim * sizeof(float));
            }
        }
        free(kd); free(vd); free(work);
    }
}

/* The 4-bit affine product that makes qg, k, v and consumes attn_out (qwasar_gpu.h:84-103;
 * qwasar_cpu.c:21-63): y[r][o] = sum_i (scale * nibble + bias) * x[r][i], element i of output
 * row o in word i/8 at bit 4 (i % 8) of w [n, k/8], scale and bias bf16 per group of `group`
 * elements ([n, k/group]); fp32, terms added in index order. */
void orc_qmv_q4(float *y, const float *x, const uint32_t *w, const uint16_t *scales, const uint16_t *biases,
                int32_t k, int32_t n, int32_t rows, int32_t group) {
    const int32_t words = k / 8, groups = k / group;
    for (int32_t r = 0; r < rows; r++)
        for (int32_t o = 0; o < n; o++) {
            float acc = 0.0f;
            for (int32_t i = 0; i < k; i++) {
                const uint32_t nib = (w[(size_t)o * words + i / 8] >> (4 * (i % 8))) & 0xF;
                const float sc = orc_bf16_up(scales[(size_t)o * groups + i / group]);
                const float bi = orc_bf16_up(biases[(size_t)o * groups + i / group]);
                acc += (sc * (float)nib + bi) * x[(size_t)r * k + i];
            }
            y[(size_t)r * n + o] = acc;
        }
}

/* QSA block scores (qwasar_flash_cpu.c:372-397; the check of tests/test_sparse.c:392-416): for
 * row r the first (base_pos + r + 1) / ratio blocks of `ratio` raw index keys each are mean-pooled
 * (sum in position order, then / ratio), RMS-normed with weight k_norm, rotated at the block's
 * first position (all three axes equal, so only inv_freq matters), and scored against the row's
 * nq normed + rotated query heads: sum over heads of max(dot, 0), / sqrt(d).  scores is
 * [rows, max_blocks]; entries of blocks not yet complete are left alone.  pool (optional,
 * [max_blocks, d]) receives the block keys. */
void orc_qsa_scores(float *scores, float *pool, const float *qn, const float *ikeys, const uint16_t *k_norm,
                    const float *inv_freq, int32_t rows, int32_t nq, int32_t d, int32_t ratio, int32_t base_pos,
                    int32_t rotary_dim, int32_t max_blocks, float eps) {
    uint8_t axis[128];
    memset(axis, 0, sizeof axis);
    float *pooled = (float *)malloc((size_t)d * sizeof(float));
    float *kn = (float *)malloc((size_t)d * sizeof(float));
    const int32_t all = (base_pos + rows) / ratio;
    float *keys = (float *)malloc((size_t)(all ? all : 1) * d * sizeof(float));
    for (int32_t b = 0; b < all; b++) {
        for (int32_t i = 0; i < d; i++) {
            float acc = 0.0f;
            for (int32_t t = 0; t < ratio; t++) acc += ikeys[(size_t)(b * ratio + t) * d + i];
            pooled[i] = acc / (float)ratio;
        }
        orc_rms_norm(kn, pooled, k_norm, d, 1, eps, 1.0f);
        const int32_t bp[3] = { b * ratio, b * ratio, b * ratio };
        orc_rope_partial(kn, bp, axis, inv_freq, 1, 1, d, rotary_dim);
        memcpy(keys + (size_t)b * d, kn, (size_t)d * sizeof(float));
        if (pool) memcpy(pool + (size_t)b * d, kn, (size_t)d * sizeof(float));
    }
    for (int32_t r = 0; r < rows; r++) {
        const int32_t n_blocks = (base_pos + r + 1) / ratio;
        for (int32_t b = 0; b < n_blocks && b < max_blocks; b++) {
            float s = 0.0f;
            for (int32_t h = 0; h < nq; h++) {
                float dot = 0.0f;
                for (int32_t i = 0; i < d; i++) dot += qn[((size_t)r * nq + h) * d + i] * keys[(size_t)b * d + i];
                if (dot > 0.0f) s += dot;
            }
            scores[(size_t)r * max_blocks + b] = s / sqrtf((float)d);
        }
    }
    free(pooled); free(kn); free(keys);
}

/* QSA selection (qwasar_flash_cpu.c:363-406; tests/test_sparse.c:452-470): row r sees positions
 * [0, base_pos + r]; the incomplete trailing block is always visible, and of the complete blocks
 * the block_topk best by score, found one at a time -- the largest score above -FLT_MAX, the
 * lowest index among equals.  mask is [rows, max_ctx] bytes (only positions [0, n_keys) of a row
 * are written), list [rows, 1 + block_topk * ratio + ratio] uint32: the count, then the visible
 * positions ascending (qwasar_gpu.h:632-639). */
void orc_qsa_select(uint8_t *mask, uint32_t *list, const float *scores, int32_t rows, int32_t ratio, int32_t base_pos,
                    int32_t block_topk, int32_t max_ctx, int32_t max_blocks) {
    const int32_t stride = 1 + block_topk * ratio + ratio;
    for (int32_t r = 0; r < rows; r++) {
        const int32_t n_keys = base_pos + r + 1, n_blocks = n_keys / ratio;
        uint8_t *m = mask + (size_t)r * max_ctx;
        for (int32_t t = 0; t < n_keys; t++) m[t] = t >= n_blocks * ratio;
        float *s = (float *)malloc((size_t)(n_blocks ? n_blocks : 1) * sizeof(float));
        memcpy(s, scores + (size_t)r * max_blocks, (size_t)n_blocks * sizeof(float));
        const int32_t take = block_topk < n_blocks ? block_topk : n_blocks;
        for (int32_t n = 0; n < take; n++) {
            int32_t best = -1;
            for (int32_t b = 0; b < n_blocks; b++)
                if (s[b] > -FLT_MAX && (best < 0 || s[b] > s[best])) best = b;
            if (best < 0) break;
            for (int32_t t = 0; t < ratio; t++) m[best * ratio + t] = 1;
            s[best] = -FLT_MAX;
        }
        free(s);
        uint32_t *l = list + (size_t)r * stride;
        uint32_t cnt = 0;
        for (int32_t t = 0; t < n_keys; t++) if (m[t]) l[1 + cnt++] = (uint32_t)t;
        l[0] = cnt;
    }
}

/* out[i] *= 1 / (1 + exp(-gate[i]))  (metal/act.metal:29-37). */
void orc_mul_sigmoid(float *y, const float *gate, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] *= 1.0f / (1.0f + expf(-gate[i]));
}

/* Un-normalised partial softmax of one (row, query head) over cache positions
 * [t0, t1): the running max m, the sum l of exp(s - m) and acc_i = sum_t
 * exp(s_t - m) V[t][i] -- the triple the split kernels leave per slice
 * (metal/attn.metal:198-259 writes exactly these as pacc/pstat).  An empty
 * range gives m = -FLT_MAX, l = 0, acc = 0. */
void orc_attn_partial(float *acc, float *stat, const float *q,
                      const uint16_t *kh, const uint16_t *vh, int32_t t0,
                      int32_t t1, int32_t head_dim, float scale, int fmt) {
    float top = -FLT_MAX;
    const int32_t n = t1 > t0 ? t1 - t0 : 0;
    float *s = (float *)malloc((size_t)(n ? n : 1) * sizeof(float));
    for (int32_t t = 0; t < n; t++) {
        const uint16_t *kr = kh + (size_t)(t0 + t) * head_dim;
        float dot = 0.0f;
        for (int32_t i = 0; i < head_dim; i++) dot += q[i] * scale * orc_cache_up(kr[i], fmt);
        s[t] = dot;
        if (dot > top) top = dot;
    }
    float l = 0.0f;
    for (int32_t i = 0; i < head_dim; i++) acc[i] = 0.0f;
    for (int32_t t = 0; t < n; t++) {
        const float e = expf(s[t] - top);
        const uint16_t *vr = vh + (size_t)(t0 + t) * head_dim;
        l += e;
        for (int32_t i = 0; i < head_dim; i++) acc[i] += e * orc_cache_up(vr[i], fmt);
    }
    stat[0] = top;
    stat[1] = l;
    free(s);
}

/* Log-sum-exp merge of `parts` partials of one (row, query head)
 * (metal/attn.metal:273-303): m = max over parts with l > 0, w_p =
 * exp(m_p - m) for live parts else 0, out_i = (sum_p acc_p[i] w_p) /
 * (sum_p l_p w_p), zero when nothing was live.  gate (may be NULL) applies
 * the sigmoid output gate as the merged value is written (:317-331).
 * pacc is [parts, head_dim], pstat is [parts, 2] = (max, sum). */
void orc_attn_merge(float *out, const float *pacc, const float *pstat,
                    int32_t parts, int32_t head_dim, const float *gate) {
    float m = -FLT_MAX;
    for (int32_t p = 0; p < parts; p++)
        if (pstat[2 * p + 1] > 0.0f && pstat[2 * p] > m) m = pstat[2 * p];
    float denom = 0.0f;
    for (int32_t i = 0; i < head_dim; i++) out[i] = 0.0f;
    for (int32_t p = 0; p < parts; p++) {
        const float l = pstat[2 * p + 1];
        const float w = l > 0.0f ? expf(pstat[2 * p] - m) : 0.0f;
        denom += l * w;
        for (int32_t i = 0; i < head_dim; i++) out[i] += pacc[(size_t)p * head_dim + i] * w;
    }
    for (int32_t i = 0; i < head_dim; i++) {
        float v = denom > 0.0f ? out[i] / denom : 0.0f;
        if (gate) v *= 1.0f / (1.0f + expf(-gate[i]));
        out[i] = v;
    }
}

/* ---- the composed node ---------------------------------------------------- */

/* The attention node in the order the graph encodes it
 * (qwasar_graph.c:630-659): split [q|gate] -> RMS norm of q and k -> partial
 * RoPE of q and k -> append K,V -> causal attention -> sigmoid gate.
 *
 *   qg   f32 [rows, q_heads, 2*head_dim]   k, v  f32 [rows, kv_heads, head_dim]
 *   qw, kw   bf16 norm weights [head_dim] or NULL
 *   pos  int32 [3, rows]; axis, inv_freq from orc_rope_tables
 *   kc, vc   head-major cache of this layer, updated in place
 *   out  f32 [rows, q_heads, head_dim]
 *   q_post (optional) receives the normed + roped query, k_post the normed +
 *   roped key -- the fp32 values that went into the attention and the append. */
void orc_attn_layer(float *out, const float *qg, const float *k, const float *v,
                    const uint16_t *qw, const uint16_t *kw, const int32_t *pos,
                    const uint8_t *axis, const float *inv_freq,
                    uint16_t *kc, uint16_t *vc, int32_t rows, int32_t q_heads,
                    int32_t kv_heads, int32_t head_dim, int32_t rotary_dim,
                    int32_t max_ctx, int32_t base_pos, float eps, float scale,
                    int fmt, int threads, float *q_post, float *k_post) {
    const size_t qn = (size_t)rows * q_heads * head_dim;
    const size_t kn = (size_t)rows * kv_heads * head_dim;
    float *qv = (float *)malloc(qn * sizeof(float));
    float *gv = (float *)malloc(qn * sizeof(float));
    float *kk = (float *)malloc(kn * sizeof(float));

    orc_split_heads2(qv, gv, qg, rows, q_heads, head_dim);
    orc_rms_norm(qv, qv, qw, head_dim, rows * q_heads, eps, 1.0f);
    orc_rms_norm(kk, k, kw, head_dim, rows * kv_heads, eps, 1.0f);
    orc_rope_partial(qv, pos, axis, inv_freq, rows, q_heads, head_dim, rotary_dim);
    orc_rope_partial(kk, pos, axis, inv_freq, rows, kv_heads, head_dim, rotary_dim);
    orc_kv_write(kc, vc, kk, v, rows, kv_heads, head_dim, max_ctx, base_pos, fmt);
    orc_attn_decode(out, qv, kc, vc, rows, q_heads, kv_heads, head_dim, max_ctx,
                    base_pos, scale, fmt, threads);
    orc_mul_sigmoid(out, gv, qn);

    if (q_post) memcpy(q_post, qv, qn * sizeof(float));
    if (k_post) memcpy(k_post, kk, kn * sizeof(float));
    free(qv); free(gv); free(kk);
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
