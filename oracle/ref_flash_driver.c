/* ref_flash_driver.c -- TEST INFRASTRUCTURE, not part of the product.
 *
 * Makes the reference's own block selection and composed gated-attention layer callable from
 * the tests: qsa_select (qwasar_flash_cpu.c:346-418) and qsa_step (:422-488) are `static` there
 * and work on the engine's bound tensors, so this file includes the reference source from where
 * it lies (oracle/Makefile passes -I to the checkout; nothing is copied), supplies the few engine
 * accessors that file links against, and builds one synthetic layer -- 4-bit affine projections,
 * norm weights -- from arrays the caller passes.  The checker then holds this repo's restatement
 * (orc_qsa_scores / orc_qsa_select / orc_attn_layer) to what these functions return. */
#include "qwasar_flash_cpu.c"

#include <stdarg.h>

/* ---- what qwasar_flash_cpu.c expects from the engine and the backend ---- */
struct qw_buf_s { void *p; };
void *qw_buf_contents(qw_buf b) { return b ? b->p : NULL; }
const void *qw_tensor_data(const qw_tensor *t) { return t->cpu ? t->cpu : (const char *)t->buf->p + t->offset; }
const qw_config *qwasar_engine_config(const qwasar_engine *e) { (void)e; return NULL; }
const qw_shape *qwasar_engine_shape(const qwasar_engine *e) { (void)e; return NULL; }
const qw_layer *qwasar_engine_layer(const qwasar_engine *e, int i) { (void)e; (void)i; return NULL; }
const qw_qlinear *qwasar_engine_embed(const qwasar_engine *e) { (void)e; return NULL; }
const qw_qlinear *qwasar_engine_head(const qwasar_engine *e) { (void)e; return NULL; }
const qw_hc *qwasar_engine_final_hc(const qwasar_engine *e) { (void)e; return NULL; }
void qw_verrf(char *err, size_t cap, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    if (err && cap) vsnprintf(err, cap, fmt, ap);
    va_end(ap);
}

/* ---- one synthetic attention layer ---- */
typedef struct {
    qw_config c;
    qw_shape sh;
    qw_layer L;
    ref_layer l;
    struct qw_flash_ref r;
    struct qw_buf_s bufs[20];
    qw_tensor tens[20];
    int n_t;
} flash_layer;

static const qw_tensor *bind(flash_layer *f, const void *data) {
    if (!data) return NULL;
    const int i = f->n_t++;
    f->bufs[i].p = (void *)data;
    memset(&f->tens[i], 0, sizeof f->tens[i]);
    f->tens[i].buf = &f->bufs[i];
    return &f->tens[i];
}
static void qlinear(flash_layer *f, qw_qlinear *q, const void *const *wsb, int in, int out, int group) {
    q->weight = bind(f, wsb[0]); q->scales = bind(f, wsb[1]); q->biases = bind(f, wsb[2]);
    q->in_features = in; q->out_features = out; q->group_size = group;
}

/* proj: five (weight U32, scales bf16, biases bf16) triples -- q_proj [q_heads*2*head_dim, hidden],
 * k_proj, v_proj [kv_heads*head_dim, hidden], o_proj [hidden_out, q_heads*head_dim], indexer
 * qk_proj [(idx_heads+1)*idx_dim, hidden]; norms: q_norm, k_norm [head_dim], indexer q_norm, k_norm
 * [idx_dim] (bf16, may be NULL).  The arrays must outlive the layer. */
void *qwflash_new(int hidden, int hidden_out, int q_heads, int kv_heads, int head_dim, int rotary_dim, float theta,
                  const int32_t *mrope_section, int idx_heads, int idx_dim, int budget, int ratio, float eps, int max_ctx,
                  int group, const void *const *proj, const void *const *norms) {
    flash_layer *f = calloc(1, sizeof *f);
    qw_config *c = &f->c;
    c->hidden_size = hidden; c->num_attention_heads = q_heads; c->num_key_value_heads = kv_heads; c->head_dim = head_dim;
    c->rms_norm_eps = eps; c->rotary_dim = rotary_dim;
    c->indexer_n_heads = idx_heads; c->indexer_kv_heads = 1; c->indexer_head_dim = idx_dim;
    c->indexer_budget = budget; c->indexer_compress_ratio = ratio;
    f->sh.q_dim = q_heads * head_dim; f->sh.q_proj_out = 2 * q_heads * head_dim; f->sh.kv_dim = kv_heads * head_dim;
    f->sh.gqa_factor = q_heads / kv_heads;
    qlinear(f, &f->L.q_proj, proj + 0, hidden, f->sh.q_proj_out, group);
    qlinear(f, &f->L.k_proj, proj + 3, hidden, f->sh.kv_dim, group);
    qlinear(f, &f->L.v_proj, proj + 6, hidden, f->sh.kv_dim, group);
    qlinear(f, &f->L.o_proj, proj + 9, f->sh.q_dim, hidden_out, group);
    qlinear(f, &f->L.indexer.qk_proj, proj + 12, hidden, (idx_heads + 1) * idx_dim, group);
    f->L.q_norm = bind(f, norms[0]); f->L.k_norm = bind(f, norms[1]);
    f->L.indexer.q_norm = bind(f, norms[2]); f->L.indexer.k_norm = bind(f, norms[3]);
    f->l.kc = calloc((size_t)max_ctx * f->sh.kv_dim, sizeof(float));
    f->l.vc = calloc((size_t)max_ctx * f->sh.kv_dim, sizeof(float));
    f->l.ikeys = calloc((size_t)max_ctx * idx_dim, sizeof(float));
    f->r.c = c; f->r.sh = &f->sh; f->r.max_ctx = max_ctx; f->r.L = &f->l;
    qw_rope_tables(f->r.axis, f->r.inv_freq, rotary_dim, theta, mrope_section);
    return f;
}
void qwflash_free(void *h) {
    flash_layer *f = h;
    if (!f) return;
    free(f->l.kc); free(f->l.vc); free(f->l.ikeys); free(f);
}
/* The reference's selection for the token at `pos` (positions must be fed in order: each call
 * stores the token's raw index key).  allowed: pos + 1 bytes.  qk: what the indexer projection
 * returned for x, (idx_heads + 1) * idx_dim floats -- the queries, then the raw key. */
void qwflash_select(void *h, const float *x, int pos, uint8_t *allowed, float *qk) {
    flash_layer *f = h;
    qsa_select(&f->r, &f->L, &f->l, x, pos, allowed);
    qlin(qk, x, &f->L.indexer.qk_proj);
}
/* The reference's whole gated attention layer for the token at `pos` (in order): out is o_proj's
 * output; qg, k, v receive what the three projections returned for x. */
void qwflash_step(void *h, const float *x, int pos, float *out, float *qg, float *k, float *v) {
    flash_layer *f = h;
    qsa_step(&f->r, &f->L, &f->l, x, pos, out);
    qlin(qg, x, &f->L.q_proj); qlin(k, x, &f->L.k_proj); qlin(v, x, &f->L.v_proj);
}
