/* The reference's attention node, written in C99 against include/qwasar_cuda.h exactly the way
 * qw_encode_attention_layer encodes it (qwasar_graph.c:619-662: split -> norm q, k -> rope q, k ->
 * kv_write -> attn -> gate, buffers from qw_buf_alloc read and written through qw_buf_contents,
 * the layer's cache addressed by byte offset), and the same node as the one fused call.  Both are
 * checked against the oracle's composition of the reference functions (oracle/qw_attn_oracle.c),
 * the way tests/test_attn.c:106-138 checks the reference's kernels against qw_cpu_attn_decode.
 *
 * This file is also the compile-and-link check of the header from plain C: -std=c99 -pedantic,
 * every declared entry point referenced.  Without a CUDA device qw_gpu_init fails with a message;
 * the program then prints it and exits 0 ("no device" is not a failure of the ABI).
 *
 *   attn_node [rows qh kvh base layers]     default: 3 24 4 200 2 (layer 1 is used)
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "qwasar_cuda.h"

/* oracle (test infrastructure only) */
void orc_rope_tables(uint8_t *axis, float *inv_freq, int32_t rotary_dim, float theta, const int32_t *mrope_section);
void orc_attn_layer(float *out, const float *qg, const float *k, const float *v, const uint16_t *qw, const uint16_t *kw,
                    const int32_t *pos, const uint8_t *axis, const float *inv_freq, uint16_t *kc, uint16_t *vc, int32_t rows,
                    int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t rotary_dim, int32_t max_ctx, int32_t base_pos,
                    float eps, float scale, int fmt, int threads, float *q_post, float *k_post);

static uint64_t rng_state = 88172645463325252ull;
static float rnd(void) {                       /* xorshift64, uniform in [-1, 1) */
    rng_state ^= rng_state << 13; rng_state ^= rng_state >> 7; rng_state ^= rng_state << 17;
    return (float)((rng_state >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;
}
static uint16_t bf16_of(float f) {             /* round to nearest even */
    uint32_t u; memcpy(&u, &f, 4);
    u += 0x7FFF + ((u >> 16) & 1);
    return (uint16_t)(u >> 16);
}
static float bf16_exact(float f) { uint32_t u = (uint32_t)bf16_of(f) << 16; float g; memcpy(&g, &u, 4); return g; }

static double max_rel_err(const float *got, const float *want, size_t vectors) {
    double worst = 0.0;
    for (size_t v = 0; v < vectors; v++) {
        double mx = 0.0, df = 0.0;
        for (int i = 0; i < 256; i++) {
            const double w = fabs(want[v * 256 + i]), d = fabs((double)got[v * 256 + i] - want[v * 256 + i]);
            if (w > mx) mx = w;
            if (d > df) df = d;
        }
        if (mx > 0 && df / mx > worst) worst = df / mx;
    }
    return worst;
}

/* every entry point of the header, so that a missing definition fails the link */
typedef void (*any_fn)(void);
static const any_fn all_symbols[] = {
    (any_fn)qw_gpu_init, (any_fn)qw_gpu_shutdown, (any_fn)qw_gpu_name, (any_fn)qw_gpu_working_set_limit,
    (any_fn)qw_gpu_max_buffer_length, (any_fn)qw_buf_alloc, (any_fn)qw_buf_wrap, (any_fn)qw_buf_free,
    (any_fn)qw_buf_contents, (any_fn)qw_buf_length, (any_fn)qw_cmd_begin, (any_fn)qw_cmd_commit,
    (any_fn)qw_cmd_wait, (any_fn)qw_cmd_flush, (any_fn)qw_cmd_parallel, (any_fn)qw_cmd_free,
    (any_fn)qw_cmd_error, (any_fn)qw_prof_enabled, (any_fn)qw_prof_report, (any_fn)qw_prof_reset, (any_fn)qw_cmd_mark, (any_fn)qw_op_split_heads2,
    (any_fn)qw_op_rms_norm, (any_fn)qw_op_rope_partial, (any_fn)qw_rope_tables, (any_fn)qw_op_kv_write, (any_fn)qw_op_slice_rows,
    (any_fn)qw_op_attn, (any_fn)qw_op_attn_decode, (any_fn)qw_op_attn_prefill, (any_fn)qw_op_attn_prefill_as,
    (any_fn)qw_op_attn_decode_split, (any_fn)qw_op_attn_decode_tensor, (any_fn)qw_op_mul_sigmoid,
    (any_fn)qw_op_attn_masked, (any_fn)qw_op_attn_masked_gated, (any_fn)qw_op_qsa_scores, (any_fn)qw_op_qsa_pool,
    (any_fn)qw_op_qsa_scores_pooled, (any_fn)qw_op_qsa_select, (any_fn)qw_op_qmat_q4, (any_fn)qw_op_qmv_q4,
    (any_fn)qw_op_qmm_q4, (any_fn)qw_op_qmv_q4_multi,
    (any_fn)qw_gpu_last_error, (any_fn)qw_gpu_sm_count, (any_fn)qw_gpu_launch_count, (any_fn)qw_gpu_tune,
    (any_fn)qw_attn_split_plan, (any_fn)qw_prof_kernels, (any_fn)qw_prof_kernel_read,
    (any_fn)qw_buf_alloc_device, (any_fn)qw_buf_wrap_device, (any_fn)qw_buf_device_ptr, (any_fn)qw_buf_upload,
    (any_fn)qw_buf_download, (any_fn)qw_cmd_begin_on_stream, (any_fn)qw_op_copy, (any_fn)qw_kv_arena_alloc,
    (any_fn)qw_kv_arena_alloc_ex, (any_fn)qw_kv_read, (any_fn)qw_kv_store, (any_fn)qw_kv_state_bytes, (any_fn)qw_kv_element_tag,
    (any_fn)qw_kv_pack, (any_fn)qw_kv_unpack, (any_fn)qw_kv_arena_trim, (any_fn)qw_kv_arena_pages_in_use,
    (any_fn)qw_kv_arena_bytes_committed, (any_fn)qw_op_attn_layer_fused, (any_fn)qw_op_attn_layer_fused_batch,
    (any_fn)qw_op_attn_batch, (any_fn)qw_op_attn_partial, (any_fn)qw_op_attn_merge, (any_fn)qw_op_attn_preop,
    (any_fn)qw_attn_decode_noalloc, (any_fn)qw_attn_decode_noalloc_scratch_bytes, (any_fn)qw_attn_decode_noalloc_status,
    (any_fn)qw_gpu_device_count, (any_fn)qw_gpu_init_multi, (any_fn)qw_gpu_select, (any_fn)qw_gpu_current,
    (any_fn)qw_kv_pool_alloc, (any_fn)qw_kv_arena_alloc_in, (any_fn)qw_kv_pool_bytes_committed,
    (any_fn)qw_xchg_create, (any_fn)qw_xchg_free, (any_fn)qw_xchg_handle_bytes, (any_fn)qw_xchg_export,
    (any_fn)qw_xchg_attach, (any_fn)qw_xchg_attach_local, (any_fn)qw_xchg_set_timeout_ms, (any_fn)qw_op_attn_exchange, (any_fn)qw_op_attn_exchange_batch,
};

int main(int argc, char **argv) {
    const int32_t rows = argc > 1 ? atoi(argv[1]) : 3, qh = argc > 2 ? atoi(argv[2]) : 24, kvh = argc > 3 ? atoi(argv[3]) : 4;
    const int32_t base = argc > 4 ? atoi(argv[4]) : 200, layers = argc > 5 ? atoi(argv[5]) : 2;
    const int32_t hd = 256, rot = 64, ctx = base + rows + 9, layer = layers - 1;
    const float eps = 1e-6f, scale = 0.0625f;
    printf("entry points referenced: %d\n", (int)(sizeof all_symbols / sizeof all_symbols[0]));

    char err[256] = "";
    if (!qw_gpu_init(err, sizeof err)) { printf("qw_gpu_init: %s\n", err); return 0; }
    printf("device: %s\n", qw_gpu_name());

    const size_t nq = (size_t)rows * qh * hd, nk = (size_t)rows * kvh * hd, kv_stride = (size_t)kvh * ctx * hd;
    /* session buffers, as qw_alloc_all makes them (qwasar_graph.c:79-111) */
    qw_buf qg = qw_buf_alloc(nq * 2 * 4), q = qw_buf_alloc(nq * 4), gate = qw_buf_alloc(nq * 4), k = qw_buf_alloc(nk * 4);
    qw_buf v = qw_buf_alloc(nk * 4), attn_out = qw_buf_alloc(nq * 4), fused_out = qw_buf_alloc(nq * 4);
    qw_buf positions = qw_buf_alloc((size_t)3 * rows * 4), rope_axis = qw_buf_alloc(32), rope_inv = qw_buf_alloc(32 * 4);
    qw_buf norm_w = qw_buf_alloc(2 * 256 * 2);
    qw_buf kcache = qw_buf_alloc(kv_stride * layers * 2), vcache = qw_buf_alloc(kv_stride * layers * 2);
    qw_buf karena = qw_kv_arena_alloc(layers, kvh, ctx, hd), varena = qw_kv_arena_alloc(layers, kvh, ctx, hd);
    if (!qg || !q || !gate || !k || !v || !attn_out || !fused_out || !positions || !rope_axis || !rope_inv || !norm_w || !kcache ||
        !vcache || !karena || !varena) { printf("FAIL: allocation: %s\n", qw_gpu_last_error()); return 1; }

    float *qg_h = (float *)qw_buf_contents(qg), *k_h = (float *)qw_buf_contents(k), *v_h = (float *)qw_buf_contents(v);
    for (size_t i = 0; i < nq * 2; i++) qg_h[i] = bf16_exact(rnd() * 1.7f);
    for (size_t i = 0; i < nk; i++) { k_h[i] = bf16_exact(rnd() * 1.7f); v_h[i] = bf16_exact(rnd() * 1.7f); }
    uint16_t *w_h = (uint16_t *)qw_buf_contents(norm_w);
    for (int i = 0; i < 512; i++) w_h[i] = bf16_of(1.0f + 0.25f * rnd());
    int32_t *pos_h = (int32_t *)qw_buf_contents(positions);
    for (int a = 0; a < 3; a++) for (int r = 0; r < rows; r++) pos_h[a * rows + r] = base + r;     /* text: all axes = position */
    const int32_t section[3] = {11, 11, 10};
    qw_rope_tables((uint8_t *)qw_buf_contents(rope_axis), (float *)qw_buf_contents(rope_inv), rot, 1e7f, section);
    /* history of the layer, in both caches and in the oracle's copy */
    uint16_t *kc_h = (uint16_t *)qw_buf_contents(kcache) + kv_stride * layer, *vc_h = (uint16_t *)qw_buf_contents(vcache) + kv_stride * layer;
    uint16_t *kc_o = (uint16_t *)calloc(kv_stride, 2), *vc_o = (uint16_t *)calloc(kv_stride, 2);
    uint16_t *hist = (uint16_t *)malloc((size_t)base * hd * 2 + 2);
    memset(qw_buf_contents(kcache), 0, kv_stride * layers * 2); memset(qw_buf_contents(vcache), 0, kv_stride * layers * 2);
    for (int h = 0; h < kvh; h++) {
        for (int kv = 0; kv < 2; kv++) {
            for (size_t i = 0; i < (size_t)base * hd; i++) hist[i] = bf16_of(rnd() * 1.7f);
            memcpy((kv ? vc_h : kc_h) + (size_t)h * ctx * hd, hist, (size_t)base * hd * 2);
            memcpy((kv ? vc_o : kc_o) + (size_t)h * ctx * hd, hist, (size_t)base * hd * 2);
            if (base && !qw_kv_store(kv ? varena : karena, layer, h, 0, base, hist, kvh, ctx, hd)) { printf("FAIL: qw_kv_store: %s\n", qw_gpu_last_error()); return 1; }
        }
    }

    /* ---- the node as the reference's graph encodes it (qwasar_graph.c:630-659) ---- */
    const qw_ref q_norm = qw_ref_at(norm_w, 0), k_norm = qw_ref_at(norm_w, 512);
    qw_cmd c = qw_cmd_begin();
    qw_op_split_heads2(c, qw_ref_at(q, 0), qw_ref_at(gate, 0), qw_ref_at(qg, 0), rows, qh, hd);
    qw_op_rms_norm(c, qw_ref_at(q, 0), qw_ref_at(q, 0), q_norm, hd, rows * qh, eps, 1.0f);
    qw_op_rms_norm(c, qw_ref_at(k, 0), qw_ref_at(k, 0), k_norm, hd, rows * kvh, eps, 1.0f);
    qw_op_rope_partial(c, qw_ref_at(q, 0), qw_ref_at(positions, 0), qw_ref_at(rope_axis, 0), qw_ref_at(rope_inv, 0), rows, qh, hd, rot);
    qw_op_rope_partial(c, qw_ref_at(k, 0), qw_ref_at(positions, 0), qw_ref_at(rope_axis, 0), qw_ref_at(rope_inv, 0), rows, kvh, hd, rot);
    const qw_ref kc_ref = qw_ref_at(kcache, kv_stride * layer * sizeof(uint16_t)), vc_ref = qw_ref_at(vcache, kv_stride * layer * sizeof(uint16_t));
    qw_op_kv_write(c, kc_ref, vc_ref, qw_ref_at(k, 0), qw_ref_at(v, 0), rows, kvh, hd, ctx, base);
    qw_op_attn(c, qw_ref_at(attn_out, 0), qw_ref_at(q, 0), kc_ref, vc_ref, rows, qh, kvh, hd, ctx, base, scale);
    qw_op_mul_sigmoid(c, qw_ref_at(attn_out, 0), qw_ref_at(gate, 0), (int64_t)nq);
    qw_cmd_commit(c);
    qw_cmd_wait(c);
    if (qw_cmd_error(c)) { printf("FAIL: GPU error: %s\n", qw_cmd_error(c)); return 1; }
    qw_cmd_free(c);

    /* ---- the same node as one call, on the paged arena (k was normed in place above: fresh copy) ---- */
    rng_state = 88172645463325252ull;
    for (size_t i = 0; i < nq * 2; i++) qg_h[i] = bf16_exact(rnd() * 1.7f);
    for (size_t i = 0; i < nk; i++) { k_h[i] = bf16_exact(rnd() * 1.7f); v_h[i] = bf16_exact(rnd() * 1.7f); }
    float *k_in = (float *)malloc(nk * 4); memcpy(k_in, k_h, nk * 4);
    c = qw_cmd_begin();
    const bool ok = qw_op_attn_layer_fused(c, qw_ref_at(fused_out, 0), qw_ref_at(qg, 0), qw_ref_at(k, 0), qw_ref_at(v, 0), q_norm, k_norm,
                                           qw_ref_at(positions, 0), qw_ref_at(rope_axis, 0), qw_ref_at(rope_inv, 0),
                                           qw_ref_at(karena, kv_stride * layer * sizeof(uint16_t)), qw_ref_at(varena, kv_stride * layer * sizeof(uint16_t)),
                                           rows, qh, kvh, hd, rot, ctx, base, eps, scale, QW_F32);
    qw_cmd_wait(c);
    if (!ok || qw_cmd_error(c)) { printf("FAIL: fused node: %s\n", qw_cmd_error(c) ? qw_cmd_error(c) : "declined"); return 1; }
    qw_cmd_free(c);

    /* ---- oracle ---- */
    float *want = (float *)malloc(nq * 4);
    uint8_t axis_o[32]; float inv_o[32];
    orc_rope_tables(axis_o, inv_o, rot, 1e7f, section);
    if (memcmp(axis_o, qw_buf_contents(rope_axis), 32) || memcmp(inv_o, qw_buf_contents(rope_inv), 128)) { printf("FAIL: rope tables differ from the oracle's\n"); return 1; }
    orc_attn_layer(want, qg_h, k_in, v_h, w_h, w_h + 256, pos_h, axis_o, inv_o, kc_o, vc_o, rows, qh, kvh, hd, rot, ctx, base, eps, scale,
                   0 /* bf16 cache */, 0, NULL, NULL);
    const double e1 = max_rel_err((const float *)qw_buf_contents(attn_out), want, (size_t)rows * qh);
    const double e2 = max_rel_err((const float *)qw_buf_contents(fused_out), want, (size_t)rows * qh);
    /* the appended V rows are one rounding of the input: bit-exact in both caches */
    int v_ok = 1;
    uint16_t *row_buf = (uint16_t *)malloc((size_t)rows * hd * 2);
    for (int h = 0; h < kvh && v_ok; h++) {
        v_ok = memcmp(vc_h + ((size_t)h * ctx + base) * hd, vc_o + ((size_t)h * ctx + base) * hd, (size_t)rows * hd * 2) == 0 &&
               qw_kv_read(varena, layer, h, base, rows, row_buf, kvh, ctx, hd) &&
               memcmp(row_buf, vc_o + ((size_t)h * ctx + base) * hd, (size_t)rows * hd * 2) == 0;
    }
    printf("op sequence: max rel err %.3e   fused node: max rel err %.3e   appended V bit-exact: %s   kernels launched: %llu\n", e1, e2,
           v_ok ? "yes" : "NO", (unsigned long long)qw_gpu_launch_count());
    const int pass = e1 <= 1e-2 && e2 <= 1e-2 && v_ok;       /* tolerance: max rel err per output vector <= 1e-2 */
    qw_buf all[] = {qg, q, gate, k, v, attn_out, fused_out, positions, rope_axis, rope_inv, norm_w, kcache, vcache, karena, varena};
    for (size_t i = 0; i < sizeof all / sizeof all[0]; i++) qw_buf_free(all[i]);
    free(want); free(kc_o); free(vc_o); free(hist); free(k_in); free(row_buf);
    qw_gpu_shutdown();
    printf(pass ? "PASS\n" : "FAIL\n");
    return pass ? 0 : 1;
}
