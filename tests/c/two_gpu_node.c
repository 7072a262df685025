/* One C99 host thread driving SEVERAL GPUs through include/qwasar_cuda.h: a sequence whose
 * positions are split over the devices of this process (qw_gpu_init_multi), each device holding
 * only its own range of the cache in an arena, the ranks' softmax partials exchanged by the
 * library's own peer stores (qw_xchg_*, qw_op_attn_exchange) and merged on every device -- the
 * multi-GPU form of the decode node for one long sequence.  Every device must end with the whole
 * gated output; it is checked against the oracle's composition of the reference functions
 * (oracle/qw_attn_oracle.c), like tests/c/attn_node.c.
 *
 * The host encodes device after device and waits only after every device's kernels are queued: the
 * kernels of different GPUs wait for each other's records, so no call may block in between.
 *
 *   two_gpu_node [devices base q_heads kv_heads]     default: 2 3000 16 2
 * With fewer devices than asked for it says so and exits 0. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "qwasar_cuda.h"

void orc_rope_tables(uint8_t *axis, float *inv_freq, int32_t rotary_dim, float theta, const int32_t *mrope_section);
void orc_attn_layer(float *out, const float *qg, const float *k, const float *v, const uint16_t *qw, const uint16_t *kw,
                    const int32_t *pos, const uint8_t *axis, const float *inv_freq, uint16_t *kc, uint16_t *vc, int32_t rows,
                    int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t rotary_dim, int32_t max_ctx, int32_t base_pos,
                    float eps, float scale, int fmt, int threads, float *q_post, float *k_post);

static uint64_t rng_state = 0x9E3779B97F4A7C15ull;
static float rnd(void) {
    rng_state ^= rng_state << 13; rng_state ^= rng_state >> 7; rng_state ^= rng_state << 17;
    return (float)((rng_state >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;
}
static uint16_t bf16_of(float f) { uint32_t u; memcpy(&u, &f, 4); u += 0x7FFF + ((u >> 16) & 1); return (uint16_t)(u >> 16); }
static float bf16_exact(float f) { uint32_t u = (uint32_t)bf16_of(f) << 16; float g; memcpy(&g, &u, 4); return g; }

#define MAX_DEV 8
typedef struct { qw_buf qg, k, v, pos, axis, inv, w, qn, out, ka, va; qw_xchg x; qw_cmd c; int32_t lo, hi; } rank_t;

int main(int argc, char **argv) {
    const int32_t G = argc > 1 ? atoi(argv[1]) : 2, base = argc > 2 ? atoi(argv[2]) : 3000;
    const int32_t qh = argc > 3 ? atoi(argv[3]) : 16, kvh = argc > 4 ? atoi(argv[4]) : 2;
    const int32_t rows = 1, hd = 256, rot = 64, ctx = base + rows + 9, n_keys = base + rows;
    const float eps = 1e-6f, scale = 0.0625f;
    char err[256] = "";
    if (G < 1 || G > MAX_DEV) { printf("FAIL: 1 to %d devices\n", MAX_DEV); return 1; }
    if (qw_gpu_device_count() < G) { printf("needs %d CUDA devices, %d present: nothing to do\n", G, qw_gpu_device_count()); return 0; }
    if (!qw_gpu_init_multi(G, err, sizeof err)) { printf("qw_gpu_init_multi: %s\n", err); return 1; }

    /* one step's inputs and the whole history, on the host */
    const size_t nq = (size_t)rows * qh * hd, nk = (size_t)rows * kvh * hd, kv_stride = (size_t)kvh * ctx * hd;
    float *qg_h = (float *)malloc(nq * 2 * 4), *k_h = (float *)malloc(nk * 4), *v_h = (float *)malloc(nk * 4);
    for (size_t i = 0; i < nq * 2; i++) qg_h[i] = bf16_exact(rnd() * 1.7f);
    for (size_t i = 0; i < nk; i++) { k_h[i] = bf16_exact(rnd() * 1.7f); v_h[i] = bf16_exact(rnd() * 1.7f); }
    uint16_t w_h[512];
    for (int i = 0; i < 512; i++) w_h[i] = bf16_of(1.0f + 0.25f * rnd());
    uint16_t *kc_o = (uint16_t *)calloc(kv_stride, 2), *vc_o = (uint16_t *)calloc(kv_stride, 2);
    for (int h = 0; h < kvh; h++)
        for (size_t i = 0; i < (size_t)base * hd; i++) { kc_o[(size_t)h * ctx * hd + i] = bf16_of(rnd() * 1.7f); vc_o[(size_t)h * ctx * hd + i] = bf16_of(rnd() * 1.7f); }
    int32_t pos_h[3] = {base, base, base};
    const int32_t section[3] = {11, 11, 10};
    uint8_t axis_h[32]; float inv_h[32];
    qw_rope_tables(axis_h, inv_h, rot, 1e7f, section);

    /* every device: its range of the cache (64-aligned cuts), its buffers, its end of the exchange */
    rank_t R[MAX_DEV];
    const int32_t span = ((n_keys + G - 1) / G + 63) / 64 * 64;
    for (int d = 0; d < G; d++) {
        rank_t *r = &R[d];
        if (!qw_gpu_select(d)) { printf("FAIL: select %d: %s\n", d, qw_gpu_last_error()); return 1; }
        r->lo = d * span < n_keys ? d * span : n_keys;
        r->hi = (d + 1) * span < n_keys ? (d + 1) * span : n_keys;
        r->qg = qw_buf_alloc(nq * 2 * 4); r->k = qw_buf_alloc(nk * 4); r->v = qw_buf_alloc(nk * 4); r->pos = qw_buf_alloc(12);
        r->axis = qw_buf_alloc(32); r->inv = qw_buf_alloc(128); r->w = qw_buf_alloc(1024);
        r->qn = qw_buf_alloc_device(nq * 2); r->out = qw_buf_alloc(nq * 4);
        r->ka = qw_kv_arena_alloc(1, kvh, ctx, hd); r->va = qw_kv_arena_alloc(1, kvh, ctx, hd);
        r->x = qw_xchg_create(G, d, rows * qh);
        if (!r->qg || !r->k || !r->v || !r->pos || !r->axis || !r->inv || !r->w || !r->qn || !r->out || !r->ka || !r->va || !r->x) {
            printf("FAIL: allocation on device %d: %s\n", d, qw_gpu_last_error()); return 1;
        }
        memcpy(qw_buf_contents(r->qg), qg_h, nq * 2 * 4); memcpy(qw_buf_contents(r->k), k_h, nk * 4); memcpy(qw_buf_contents(r->v), v_h, nk * 4);
        memcpy(qw_buf_contents(r->pos), pos_h, 12); memcpy(qw_buf_contents(r->axis), axis_h, 32); memcpy(qw_buf_contents(r->inv), inv_h, 128);
        memcpy(qw_buf_contents(r->w), w_h, 1024);
        const int32_t h_hi = r->hi < base ? r->hi : base;
        for (int h = 0; h < kvh && h_hi > r->lo; h++)
            if (!qw_kv_store(r->ka, 0, h, r->lo, h_hi - r->lo, kc_o + ((size_t)h * ctx + r->lo) * hd, kvh, ctx, hd) ||
                !qw_kv_store(r->va, 0, h, r->lo, h_hi - r->lo, vc_o + ((size_t)h * ctx + r->lo) * hd, kvh, ctx, hd)) {
                printf("FAIL: qw_kv_store on device %d: %s\n", d, qw_gpu_last_error()); return 1;
            }
    }
    for (int a = 0; a < G; a++)
        for (int b = 0; b < G; b++)
            if (a != b && !qw_xchg_attach_local(R[a].x, b, R[b].x)) { printf("FAIL: attach: %s\n", qw_gpu_last_error()); return 1; }

    /* two steps' worth of rounds (the exchange alternates between two sets of slots): encode on every
     * device, then wait for every device */
    int pass = 1;
    float *want = (float *)malloc(nq * 4);
    orc_attn_layer(want, qg_h, k_h, v_h, w_h, w_h + 256, pos_h, axis_h, inv_h, kc_o, vc_o, rows, qh, kvh, hd, rot, ctx, base, eps, scale,
                   0 /* bf16 cache */, 0, NULL, NULL);
    for (int round = 0; round < 3 && pass; round++) {
        for (int d = 0; d < G; d++) {
            rank_t *r = &R[d];
            memset(qw_buf_contents(r->out), 0, nq * 4);
            qw_gpu_select(d);
            r->c = qw_cmd_begin();
            const bool owner = r->lo <= base && base < r->hi;       /* appends the new token's K, V */
            bool ok = qw_op_attn_preop(r->c, qw_ref_at(r->qn, 0), qw_ref_at(r->qg, 0), qw_ref_at(r->k, 0), qw_ref_at(r->v, 0), qw_ref_at(r->w, 0),
                                       qw_ref_at(r->w, 512), qw_ref_at(r->pos, 0), qw_ref_at(r->axis, 0), qw_ref_at(r->inv, 0),
                                       qw_ref_at(r->ka, 0), qw_ref_at(r->va, 0), rows, qh, kvh, hd, rot, ctx, base, eps, QW_F32, owner);
            ok = ok && qw_op_attn_exchange(r->c, r->x, 0, qw_ref_at(r->out, 0), qw_ref_at(r->qg, 256 * 4), qw_ref_at(r->qn, 0),
                                           qw_ref_at(r->ka, 0), qw_ref_at(r->va, 0), rows, qh, kvh, hd, ctx, base, r->lo, r->hi, scale,
                                           QW_BF16, QW_F32, QW_F32, 512);
            if (!ok) { printf("FAIL: encode on device %d: %s\n", d, qw_cmd_error(r->c) ? qw_cmd_error(r->c) : "declined"); return 1; }
            qw_cmd_commit(r->c);
        }
        for (int d = 0; d < G; d++) {
            rank_t *r = &R[d];
            qw_cmd_wait(r->c);
            if (qw_cmd_error(r->c)) { printf("FAIL: device %d: %s\n", d, qw_cmd_error(r->c)); return 1; }
            qw_cmd_free(r->c);
            double worst = 0.0;
            const float *got = (const float *)qw_buf_contents(r->out);
            for (size_t vct = 0; vct < (size_t)rows * qh; vct++) {
                double mx = 0.0, df = 0.0;
                for (int i = 0; i < 256; i++) {
                    const double w = fabs(want[vct * 256 + i]), e = fabs((double)got[vct * 256 + i] - want[vct * 256 + i]);
                    if (w > mx) mx = w;
                    if (e > df) df = e;
                }
                if (mx > 0 && df / mx > worst) worst = df / mx;
            }
            printf("round %d device %d (keys [%d, %d)): max rel err %.3e\n", round, d, r->lo, r->hi, worst);
            if (!(worst <= 1e-2)) pass = 0;
        }
    }
    for (int d = 0; d < G; d++) {
        rank_t *r = &R[d];
        qw_gpu_select(d);
        qw_xchg_free(r->x);
        qw_buf all[] = {r->qg, r->k, r->v, r->pos, r->axis, r->inv, r->w, r->qn, r->out, r->ka, r->va};
        for (size_t i = 0; i < sizeof all / sizeof all[0]; i++) qw_buf_free(all[i]);
    }
    qw_gpu_shutdown();
    printf(pass ? "PASS\n" : "FAIL\n");
    return pass ? 0 : 1;
}
