/* flash_ref_unit.c -- TEST INFRASTRUCTURE.  The reference's CPU forward (qwasar_flash_cpu.c,
 * included from where it lies) as one translation unit, plus a way to run ONE attention layer of
 * a loaded engine for one token: the reference's own qsa_step (qwasar_flash_cpu.c:422-488) on the
 * layer's bound weights and this reference state's caches.  flash_toy_gpu.c compares the same
 * layer, encoded by the reference's graph code on the CUDA backend, with it. */
#include "qwasar_flash_cpu.c"

/* out: hidden_size floats (o_proj's output); allowed: pos + 1 bytes, the positions the query saw.
 * Positions of one layer must be fed in order. */
void toy_ref_attn_step(qw_flash_ref *r, int layer, const float *x, int pos, float *out, uint8_t *allowed) {
    const qw_layer *L = qwasar_engine_layer(r->e, layer);
    r->cur_layer = layer;
    qsa_step(r, L, &r->L[layer], x, pos, out);
    if (allowed && r->dbg_mask) memcpy(allowed, qw_flash_ref_mask(r, layer, pos), (size_t)pos + 1);
}
