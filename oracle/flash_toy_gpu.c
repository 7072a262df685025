/* flash_toy_gpu.c -- TEST INFRASTRUCTURE.  The reference's own graph code for the Flash-Next
 * attention layer -- encode_qsa_layer (qwasar_flash_graph.c:408-511), unmodified, included from
 * where it lies -- encoding onto THIS repository's CUDA backend (libqwasar_cuda.so), with the
 * reference's engine loader binding the toy checkpoint's weights and its session code allocating
 * every buffer through the backend.  For each attention layer of the toy, tokens are fed one at a
 * time past the selection budget (dense branch, then scores -> selection -> masked gated
 * attention), then in multi-row chunks on a fresh session, and the layer's output (o_proj of the
 * gated attention) and the selected positions are held to the reference's CPU layer
 * (qsa_step, via flash_ref_unit.c) at the bound the reference's own test gives its GPU path
 * against its CPU path (5e-3 of the scale, tests/test_flashnext.c:318-321).
 *
 * The graph file also encodes the layers this backend does not implement (Gated DeltaNet, MoE,
 * hyper-connections, the engram layer); their ops are defined in flash_op_stubs.c as stubs that
 * stop the program, and are never reached: only the attention layer is encoded.
 *
 *   flash_toy_gpu <fixture directory>       prints one JSON line; exit status 0 = all held */
#include "qwasar_flash_graph.c"

#include <stdio.h>

void toy_ref_attn_step(qw_flash_ref *r, int layer, const float *x, int pos, float *out, uint8_t *allowed);

static uint32_t rng_state = 0x2545F491u;
static float rnd(void) {                     /* uniform in [-1, 1) */
    rng_state ^= rng_state << 13; rng_state ^= rng_state >> 17; rng_state ^= rng_state << 5;
    return (float)((int32_t)(rng_state >> 8) - 8388608) / 8388608.0f;
}

typedef struct { double worst; int mask_bad, steps, sparse_steps; } tally;

/* rows tokens of layer `li` at positions n_past .. through the reference's graph code on the CUDA
 * backend; x: [rows, hidden].  Output rows go to got [rows, hidden]; the selected positions of
 * every row are compared with `want_mask` rows (pos + 1 bytes each, NULL = dense). */
static bool gpu_rows(qwasar_session *s, const qw_layer *L, int li, const float *x, int rows, int n_past, float *got,
                     uint8_t *const *want_mask, tally *t) {
    const qw_config *cfg = s->cfg;
    const int H = cfg->hidden_size;
    memcpy(qw_buf_contents(s->hn), x, (size_t)rows * H * sizeof(float));
    int32_t *p = qw_buf_contents(s->positions);
    for (int a = 0; a < 3; a++)
        for (int r = 0; r < rows; r++) p[a * rows + r] = n_past + r;
    s->n_past = n_past;
    qw_cmd c = qw_cmd_begin();
    encode_qsa_layer(s, c, L, s->kind_index[li], rows);
    qw_cmd_wait(c);
    const char *e = qw_cmd_error(c);
    if (e) { fprintf(stderr, "GPU error: %s\n", e); qw_cmd_free(c); return false; }
    qw_cmd_free(c);
    memcpy(got, qw_buf_contents(s->hn2), (size_t)rows * H * sizeof(float));
    const int ratio = cfg->indexer_compress_ratio, topk = cfg->indexer_budget / ratio;
    if ((n_past + rows) / ratio > topk) {
        /* the list qw_op_qsa_select left: per row a count, then the visible positions ascending */
        const int cap = topk * ratio + ratio;
        const uint32_t *ql = qw_buf_contents(s->flash->qlist);
        for (int r = 0; r < rows; r++) {
            const int pos = n_past + r;
            uint8_t seen[512];
            memset(seen, 0, sizeof seen);
            const uint32_t cnt = ql[(size_t)r * (1 + cap)];
            for (uint32_t i = 0; i < cnt && i < (uint32_t)cap; i++) {
                const uint32_t q = ql[(size_t)r * (1 + cap) + 1 + i];
                if (q < sizeof seen) seen[q] = 1;
            }
            for (int q = 0; q <= pos; q++) t->mask_bad += (seen[q] != 0) != (want_mask[r][q] != 0);
            t->sparse_steps++;
        }
    }
    return true;
}

static void compare(const float *got, const float *want, int n, tally *t) {
    float md = 0.0f, scale = 1.0f;
    for (int i = 0; i < n; i++) {
        if (fabsf(got[i] - want[i]) > md) md = fabsf(got[i] - want[i]);
        if (fabsf(want[i]) > scale) scale = fabsf(want[i]);
    }
    if (md / scale > t->worst) t->worst = md / scale;
    t->steps++;
}

int main(int argc, char **argv) {
    if (argc < 2) { fprintf(stderr, "usage: %s <fixture dir>\n", argv[0]); return 2; }
    char err[512] = "";
    qwasar_options o;
    memset(&o, 0, sizeof o);
    o.model_path = argv[1]; o.context_size = 256;
    qwasar_engine *e = qwasar_engine_load(&o, err, sizeof err);
    if (!e) { fprintf(stderr, "load: %s\n", err); return 1; }
    const qw_config *cfg = qwasar_engine_config(e);
    const int H = cfg->hidden_size, NL = cfg->num_hidden_layers, P = 40;
    tally by_token = {0, 0, 0, 0}, by_chunk = {0, 0, 0, 0};
    int layers = 0;
    float *x = malloc((size_t)P * H * sizeof(float)), *want = malloc((size_t)P * H * sizeof(float)), *got = malloc((size_t)P * H * sizeof(float));
    uint8_t *masks[64], *mask_mem = calloc((size_t)P * 256, 1);
    for (int i = 0; i < P; i++) masks[i] = mask_mem + (size_t)i * 256;

    for (int li = 0; li < NL; li++) {
        const qw_layer *L = qwasar_engine_layer(e, li);
        if (L->is_linear_attn) continue;
        layers++;
        for (int i = 0; i < P * H; i++) x[i] = rnd();
        /* the CPU layer, token by token */
        qw_flash_ref *r = qw_flash_ref_new(e, 256);
        qw_flash_ref_debug(r, true);
        for (int pos = 0; pos < P; pos++) toy_ref_attn_step(r, li, x + (size_t)pos * H, pos, want + (size_t)pos * H, masks[pos]);
        /* the graph's layer on the CUDA backend: one token at a time ... */
        qwasar_session *s = qwasar_session_new(e, err, sizeof err);
        if (!s) { fprintf(stderr, "session: %s\n", err); return 1; }
        for (int pos = 0; pos < P; pos++) {
            if (!gpu_rows(s, L, li, x + (size_t)pos * H, 1, pos, got, &masks[pos], &by_token)) return 1;
            compare(got, want + (size_t)pos * H, H, &by_token);
        }
        qwasar_session_free(s);
        /* ... and as chunks of several rows on a fresh session (a prefill in pieces) */
        s = qwasar_session_new(e, err, sizeof err);
        if (!s) { fprintf(stderr, "session: %s\n", err); return 1; }
        static const int chunk[] = {8, 8, 5, 1, 12, 6};
        int pos = 0;
        for (size_t ci = 0; ci < sizeof chunk / sizeof *chunk; ci++) {
            const int rows = chunk[ci] < s->max_rows ? chunk[ci] : s->max_rows;
            if (!gpu_rows(s, L, li, x + (size_t)pos * H, rows, pos, got, &masks[pos], &by_chunk)) return 1;
            compare(got, want + (size_t)pos * H, rows * H, &by_chunk);
            pos += rows;
        }
        qwasar_session_free(s);
        qw_flash_ref_free(r);
    }
    const int ok = layers > 0 && by_token.worst <= 5e-3 && by_chunk.worst <= 5e-3 && !by_token.mask_bad && !by_chunk.mask_bad &&
                   by_token.sparse_steps > 0 && by_chunk.sparse_steps > 0;
    printf("{\"device\": \"%s\", \"attention_layers\": %d, \"tokens\": %d, \"token_by_token\": {\"worst_rel\": %.3e, \"mask_entries_differ\": %d, "
           "\"steps\": %d, \"steps_past_budget\": %d}, \"chunks\": {\"worst_rel\": %.3e, \"mask_entries_differ\": %d, \"calls\": %d, "
           "\"rows_past_budget\": %d}, \"ok\": %s}\n",
           qw_gpu_name(), layers, P, by_token.worst, by_token.mask_bad, by_token.steps, by_token.sparse_steps, by_chunk.worst,
           by_chunk.mask_bad, by_chunk.steps, by_chunk.sparse_steps, ok ? "true" : "false");
    qwasar_engine_free(e);
    return ok ? 0 : 1;
}
