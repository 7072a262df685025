/* Thread-parallel driver around the reference's own scalar attention, for the
 * timed CPU baseline -- TEST/BENCH INFRASTRUCTURE ONLY.
 *
 * This file is linked into oracle/_ref/ together with the object compiled from
 * the reference's unmodified qwasar_cpu.c.  It calls the untouched
 * qw_cpu_attn_decode on independent slices: one (row, query head) per call,
 * expressed through the function's own arguments (rows = 1, base_pos + r,
 * q_heads = kv_heads = 1 with offset pointers).  qwasar_cpu.c:364-389 keeps no
 * state across rows or heads, so every output element sees the arithmetic it
 * would see in a single whole call. */
#include <stdint.h>
#include <stddef.h>
#ifdef _OPENMP
#include <omp.h>
#endif

void qw_cpu_attn_decode(float *out, const float *q, const uint16_t *kc,
                        const uint16_t *vc, int32_t rows, int32_t q_heads,
                        int32_t kv_heads, int32_t head_dim, int32_t max_ctx,
                        int32_t base_pos, float scale);

void qwref_attn_decode_mt(float *out, const float *q, const uint16_t *kc,
                          const uint16_t *vc, int32_t rows, int32_t q_heads,
                          int32_t kv_heads, int32_t head_dim, int32_t max_ctx,
                          int32_t base_pos, float scale, int threads) {
    const int32_t group = q_heads / kv_heads;
    const int32_t pairs = rows * q_heads;
    (void)threads;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
#endif
    for (int32_t p = 0; p < pairs; p++) {
        const int32_t r = p / q_heads, h = p % q_heads;
        const size_t head_off = (size_t)(h / group) * max_ctx * head_dim;
        qw_cpu_attn_decode(out + (size_t)p * head_dim, q + (size_t)p * head_dim,
                           kc + head_off, vc + head_off, 1, 1, 1, head_dim,
                           max_ctx, base_pos + r, scale);
    }
}

int qwref_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
