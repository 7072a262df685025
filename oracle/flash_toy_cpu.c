/* flash_toy_cpu.c -- TEST INFRASTRUCTURE.  The reference's engine loader and CPU forward, built
 * on Linux from the reference's own sources, run on its toy checkpoint
 * (tests/fixtures/flashnext-tiny-q4) and held to that fixture's oracle.json the way the
 * reference's own test does (tests/test_flashnext.c:56-226): every layer's residual streams at
 * every position within 1e-3 of the oracle's scale, every position's logits within 2e-3, no
 * argmax flips, the same block-selection masks.  Prints one JSON line; exit status 0 = all held.
 *
 *   flash_toy_cpu <fixture directory>
 */
#include "qwasar.h"
#include "qwasar_json.h"
#include "qwasar_model.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static int32_t numbers(const qj_doc *d, const qj_node *arr, float *out, int32_t cap) {
    int32_t n = 0;
    for (const qj_node *v = qj_first(d, arr); v; v = qj_next(d, v)) {
        if (v->type == QJ_ARRAY) n += numbers(d, v, out ? out + n : NULL, cap - n);
        else if (v->type == QJ_NUMBER) { if (out && n < cap) out[n] = (float)v->u.num; n++; }
    }
    return n;
}

int main(int argc, char **argv) {
    if (argc < 2) { fprintf(stderr, "usage: %s <fixture dir>\n", argv[0]); return 2; }
    char err[512] = "", path[1024];
    qwasar_options o;
    memset(&o, 0, sizeof o);
    o.model_path = argv[1]; o.context_size = 256;
    qwasar_engine *e = qwasar_engine_load(&o, err, sizeof err);
    if (!e) { fprintf(stderr, "load: %s\n", err); return 1; }
    const qw_config *c = qwasar_engine_config(e);
    const int32_t HH = qwasar_engine_shape(e)->hc_hidden, NL = c->num_hidden_layers, vocab = c->vocab_size;

    snprintf(path, sizeof path, "%s/oracle.json", argv[1]);
    qj_doc d;
    if (!qj_parse_file(&d, path)) { fprintf(stderr, "oracle.json: %s\n", d.err); return 1; }
    const qj_node *root = qj_root(&d);
    int32_t tokens[64], n = 0;
    for (const qj_node *v = qj_first(&d, qj_get(&d, root, "tokens")); v && n < 64; v = qj_next(&d, v)) tokens[n++] = (int32_t)v->u.num;
    float *want = malloc((size_t)n * vocab * sizeof(float)), *want_h = malloc((size_t)NL * n * HH * sizeof(float));
    if (numbers(&d, qj_get(&d, root, "logits_full"), want, n * vocab) != n * vocab ||
        numbers(&d, qj_get(&d, root, "hidden_per_layer"), want_h, NL * n * HH) != NL * n * HH) { fprintf(stderr, "oracle.json: sizes\n"); return 1; }

    qw_flash_ref *r = qw_flash_ref_new(e, 256);
    qw_flash_ref_debug(r, true);
    float *got = calloc((size_t)n * vocab, sizeof(float)), *one = calloc((size_t)NL * HH, sizeof(float));
    float *got_h = calloc((size_t)NL * n * HH, sizeof(float));
    for (int32_t t = 0; t < n; t++) {
        if (!qw_flash_ref_forward(r, tokens + t, 1, got + (size_t)t * vocab, one, err, sizeof err)) { fprintf(stderr, "forward: %s\n", err); return 1; }
        for (int32_t i = 0; i < NL; i++) memcpy(got_h + ((size_t)i * n + t) * HH, one + (size_t)i * HH, (size_t)HH * sizeof(float));
    }
    /* residual streams per layer, relative to the layer's scale */
    double worst_layer = 0.0;
    int bad_layers = 0;
    for (int32_t i = 0; i < NL; i++) {
        float md = 0.0f, scale = 1.0f;
        for (int32_t j = 0; j < n * HH; j++) {
            const float a = got_h[(size_t)i * n * HH + j], b = want_h[(size_t)i * n * HH + j];
            if (fabsf(a - b) > md) md = fabsf(a - b);
            if (fabsf(b) > scale) scale = fabsf(b);
        }
        if (md / scale > worst_layer) worst_layer = md / scale;
        if (md > 1e-3f * scale) bad_layers++;
    }
    /* logits and their argmax */
    float worst_logit = 0.0f;
    int flips = 0;
    for (int32_t t = 0; t < n; t++) {
        int32_t ag = 0, aw = 0;
        for (int32_t v = 0; v < vocab; v++) {
            const float a = got[(size_t)t * vocab + v], b = want[(size_t)t * vocab + v];
            if (fabsf(a - b) > worst_logit) worst_logit = fabsf(a - b);
            if (a > got[(size_t)t * vocab + ag]) ag = v;
            if (b > want[(size_t)t * vocab + aw]) aw = v;
        }
        flips += ag != aw;
    }
    /* the block-selection masks of the attention layers */
    int mask_bad = 0, li = 0, sparse_layers = 0;
    for (const qj_node *lm = qj_first(&d, qj_get(&d, root, "masks_per_layer")); lm && li < NL; lm = qj_next(&d, lm), li++) {
        if (lm->type != QJ_ARRAY) continue;
        sparse_layers++;
        int32_t t = 0;
        for (const qj_node *tr = qj_first(&d, lm); tr && t < n; tr = qj_next(&d, tr), t++) {
            const uint8_t *m = qw_flash_ref_mask(r, li, t);
            int32_t p = 0;
            for (const qj_node *v = qj_first(&d, tr); v && p <= t; v = qj_next(&d, v), p++)
                mask_bad += ((int32_t)v->u.num != 0) != (m[p] != 0);
        }
    }
    const int ok = !bad_layers && worst_logit < 2e-3f && !flips && !mask_bad;
    printf("{\"tokens\": %d, \"layers\": %d, \"attention_layers\": %d, \"worst_layer_rel\": %.3e, \"layers_over_1e-3\": %d, "
           "\"worst_logit_abs\": %.3e, \"argmax_flips\": %d, \"mask_entries_differ\": %d, \"ok\": %s}\n",
           n, NL, sparse_layers, worst_layer, bad_layers, worst_logit, flips, mask_bad, ok ? "true" : "false");
    return ok ? 0 : 1;
}
