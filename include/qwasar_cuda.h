/* qwasar_cuda.h -- C ABI of the B200 (sm_100a) backend for qwasar's gated GQA
 * full-attention path.
 *
 * The first part re-declares, with unchanged names, argument order and
 * meaning, the subset of the reference's backend boundary (qwasar_gpu.h) that
 * the attention node uses; each declaration cites the reference declaration it
 * implements.  A translation unit that already includes the reference's
 * qwasar_gpu.h may define QWASAR_GPU_H's types first: the typedefs below are
 * skipped when QWASAR_GPU_H is defined.  The second part is additive: entry
 * points the reference does not have (device-resident buffers, the paged K/V
 * arena, the fused node, batched decode, partials for the exchange between
 * GPUs).  Plain C99; no CUDA or torch types appear in any signature.
 *
 * Cache element type: bfloat16 (the reference stores IEEE half,
 * qwasar_gpu.h:395-400).  Activations are fp32 in the reference signatures;
 * the additive entry points take a qw_dtype.
 *
 * Alignment: activation and weight operands (q, qg, k, v, out, gate, norm
 * weights, partials) must start on a 16-byte boundary of device memory, i.e.
 * qw_ref offsets that are multiples of 16 into buffers from qw_buf_alloc
 * (256-byte aligned); positions, rope axes and frequencies need only their
 * element alignment.  An op given an operand that is not declines: bool ops
 * return false, and qw_cmd_error names the operand. */
#ifndef QWASAR_CUDA_H
#define QWASAR_CUDA_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ======================================================================== *
 *  Part 1 -- the reference boundary (qwasar_gpu.h)                          *
 * ======================================================================== */

#ifndef QWASAR_GPU_H
/* qwasar_gpu.h:13-16 -- opaque buffer handle. */
typedef struct qw_buf_s *qw_buf;
/* qwasar_gpu.h:45-52 -- a tensor argument: buffer + byte offset, by value.
 * {NULL, 0} means "operand absent" (qwasar_gpu.h:269-272). */
typedef struct { qw_buf buf; size_t off; } qw_ref;
static inline qw_ref qw_ref_at(qw_buf b, size_t off) { qw_ref r = { b, off }; return r; }
static inline qw_ref qw_ref_offset(qw_ref r, size_t off) { r.off += off; return r; }
/* qwasar_gpu.h:54 -- one command buffer under construction. */
typedef struct qw_cmd_s *qw_cmd;
/* qwasar_gpu.h:105-109 -- one of the products of qw_op_qmv_q4_multi. */
typedef struct { qw_ref y, w, scales, biases; int32_t n; } qw_qmv_part;
#endif

/* qwasar_gpu.h:18-23.  Idempotent; false + message in err on failure (no
 * CUDA device, not compute capability 10.x, driver entry points missing). */
bool qw_gpu_init(char *err, size_t errcap);
void qw_gpu_shutdown(void);
/* qwasar_gpu.h:25-28. */
const char *qw_gpu_name(void);
uint64_t    qw_gpu_working_set_limit(void);   /* bytes of device memory */
uint64_t    qw_gpu_max_buffer_length(void);

/* qwasar_gpu.h:30-37.  A buffer from qw_buf_alloc is "shared": qw_buf_contents
 * returns pinned host memory the CPU reads and writes directly, mirrored in
 * device memory.  The mirror is refreshed from the host copy the first time a
 * command buffer touches a byte range, and ranges an op wrote are copied back
 * by qw_cmd_wait; so host writes must precede the encoding of the op that
 * reads them, and results are read after qw_cmd_wait -- the order every
 * caller in the reference already follows (qwasar_graph.c:1525-1570).
 * New buffers are zero-filled.  qw_buf_wrap mirrors caller-owned host memory
 * the same way (it is page-locked when the platform allows). */
qw_buf qw_buf_wrap(void *ptr, size_t len);
qw_buf qw_buf_alloc(size_t len);
void   qw_buf_free(qw_buf b);                 /* NULL-safe */
void  *qw_buf_contents(qw_buf b);             /* NULL for device-only buffers and arenas */
size_t qw_buf_length(qw_buf b);

/* qwasar_gpu.h:56-69.  One qw_cmd is one CUDA stream: ops are launched as
 * they are encoded and run in encoding order, so "each dispatch sees
 * everything before it" holds; qw_cmd_parallel regions are accepted and run
 * serially (same results).  qw_cmd_commit and qw_cmd_flush are submission
 * hints; qw_cmd_wait blocks until everything encoded has finished, copies
 * written ranges of shared buffers back to the host, and latches the first
 * error, which qw_cmd_error then returns (NULL when there was none). */
qw_cmd qw_cmd_begin(void);
void   qw_cmd_commit(qw_cmd c);
void   qw_cmd_wait(qw_cmd c);
void   qw_cmd_flush(qw_cmd c);
void   qw_cmd_parallel(qw_cmd c, bool on);
void   qw_cmd_free(qw_cmd c);
const char *qw_cmd_error(qw_cmd c);

/* qwasar_gpu.h:77-82.  QWASAR_PROFILE=1: qw_cmd_mark times the work since the
 * previous mark with a pair of CUDA events and charges it to `label`;
 * qw_prof_report prints the table to `out`, per token when tokens > 0, and
 * qw_prof_reset empties it (qwasar_metal.m:396-450). */
bool qw_prof_enabled(void);
void qw_cmd_mark(qw_cmd c, const char *label);
void qw_prof_report(FILE *out, long tokens);
void qw_prof_reset(void);

/* qwasar_gpu.h:391-393.  [rows, heads, 2*dim] f32 -> two [rows, heads, dim]. */
void qw_op_split_heads2(qw_cmd c, qw_ref a, qw_ref b, qw_ref src,
                        int32_t rows, int32_t heads, int32_t dim);
/* qwasar_gpu.h:269-276.  weight: bf16 [dim] or a null ref. */
void qw_op_rms_norm(qw_cmd c, qw_ref y, qw_ref x, qw_ref weight,
                    int32_t dim, int32_t rows, float eps, float out_scale);
/* qwasar_gpu.h:366-377.  In place; pos int32 [3, rows], axis uint8
 * [rotary_dim/2], inv_freq f32 [rotary_dim/2]. */
void qw_op_rope_partial(qw_cmd c, qw_ref x, qw_ref pos, qw_ref axis, qw_ref inv_freq,
                        int32_t rows, int32_t heads, int32_t head_dim, int32_t rotary_dim);
/* qwasar_gpu.h:379-382 (host function; qwasar_cpu.c:284-302). */
void qw_rope_tables(uint8_t *axis, float *inv_freq, int32_t rotary_dim,
                    float theta, const int32_t mrope_section[3]);
/* qwasar_gpu.h:385.  y[i] *= sigmoid(gate[i]). */
void qw_op_mul_sigmoid(qw_cmd c, qw_ref y, qw_ref gate, int32_t n);

/* qwasar_gpu.h:387-389.  dst[r, 0:len] = src[r, offset:offset+len], f32 rows of src_stride floats:
 * how the Flash-Next attention layer takes the indexer's key and query heads out of their joint
 * projection (qwasar_flash_graph.c:446-452). */
void qw_op_slice_rows(qw_cmd c, qw_ref dst, qw_ref src, int32_t rows, int32_t src_stride, int32_t offset, int32_t len);
/* qwasar_gpu.h:402-406.  Appends rows of K and V at base_pos, rounding to the
 * cache type (bf16, round-to-nearest-even).  The cache refs address one layer:
 * either a plain buffer holding the reference's head-major
 * [kv_heads, max_ctx, head_dim] array, or an arena from qw_kv_arena_alloc
 * addressed exactly as the reference addresses its cache -- byte offset
 * layer * kv_heads * max_ctx * head_dim * 2 (qwasar_graph.c:624,646-653). */
void qw_op_kv_write(qw_cmd c, qw_ref kcache, qw_ref vcache, qw_ref k, qw_ref v,
                    int32_t rows, int32_t kv_heads, int32_t head_dim,
                    int32_t max_ctx, int32_t base_pos);

/* qwasar_gpu.h:408-413.  The per-query kernel: fp32 throughout. */
void qw_op_attn_decode(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache,
                       int32_t rows, int32_t q_heads, int32_t kv_heads,
                       int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale);
/* qwasar_gpu.h:415-422.  The tiled kernel for many query rows.  Returns
 * false, encoding nothing, when head_dim != 256 or the grouping does not fit. */
bool qw_op_attn_prefill(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache,
                        int32_t rows, int32_t q_heads, int32_t kv_heads,
                        int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale);
/* qwasar_gpu.h:424-428.  half_form is accepted and ignored: this backend has
 * one form (bf16 operands, fp32 accumulation). */
bool qw_op_attn_prefill_as(qw_cmd c, bool half_form, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache,
                           int32_t rows, int32_t q_heads, int32_t kv_heads,
                           int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale);
/* qwasar_gpu.h:430-437 and :509-515.  Both names reach the same split-KV
 * tensor-op kernel, which takes any q_heads / kv_heads grouping with
 * rows * grouping <= 64 (the reference's split kernel is fixed at 6:1). */
bool qw_op_attn_decode_split(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache,
                             int32_t rows, int32_t q_heads, int32_t kv_heads,
                             int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale);
bool qw_op_attn_decode_tensor(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache,
                              int32_t rows, int32_t q_heads, int32_t kv_heads,
                              int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale);
/* qwasar_gpu.h:635-651 -- attention that sees only listed cache positions (what the QSA layers of
 * Flash-Next run once a selection exists).  list: uint32 [rows, 1 + cap] with cap = block_topk *
 * ratio + ratio (qw_qsa_list_cap, :637-639): per row a count, then that many positions ascending;
 * entries past the count are never read.  Row r of query head h attends those positions of kv head
 * h / (q_heads / kv_heads).  The gated form multiplies by sigmoid(gate), gate f32 [rows, q_heads,
 * head_dim].  fp32 throughout (CUDA cores). */
void qw_op_attn_masked(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache, qw_ref list,
                       int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                       int32_t max_ctx, int32_t base_pos, float scale, int32_t block_topk, int32_t ratio);
void qw_op_attn_masked_gated(qw_cmd c, qw_ref out, qw_ref gate, qw_ref q, qw_ref kcache, qw_ref vcache,
                             qw_ref list, int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                             int32_t max_ctx, int32_t base_pos, float scale, int32_t block_topk, int32_t ratio);
/* qwasar_gpu.h:84-118 -- the 4-bit affine product that produces qg, k, v and consumes attn_out:
 * y f32 [rows, n] = x f32 [rows, k] . dequant(w)^T, with w U32 [n, k/8] (MLX affine 4-bit: element
 * i of a row in word i/8 at bit 4 (i % 8)), scales and biases bf16 [n, k/group], group 32 or 64,
 * element = scale * nibble + bias.  The three names reach one fp32 kernel (the reference picks
 * among three by shape).  qw_op_qmv_q4_multi: up to 4 one-token products sharing x, k >= 2048,
 * else false and nothing encoded (:105-109). */
void qw_op_qmat_q4(qw_cmd c, qw_ref y, qw_ref x, qw_ref w, qw_ref scales, qw_ref biases,
                   int32_t k, int32_t n, int32_t rows, int32_t group);
void qw_op_qmv_q4(qw_cmd c, qw_ref y, qw_ref x, qw_ref w, qw_ref scales, qw_ref biases,
                  int32_t k, int32_t n, int32_t rows, int32_t group);
void qw_op_qmm_q4(qw_cmd c, qw_ref y, qw_ref x, qw_ref w, qw_ref scales, qw_ref biases,
                  int32_t k, int32_t n, int32_t rows, int32_t group);
bool qw_op_qmv_q4_multi(qw_cmd c, qw_ref x, int32_t k, int32_t group, int32_t count, const qw_qmv_part *parts);
/* qwasar_gpu.h:620-634 -- QSA's indexer.  qn f32 [rows, nq, d] are the normed + rotated index
 * queries, ikeys f32 [positions, d] a layer's raw index keys, k_norm bf16 [d] (or a null ref),
 * inv_freq f32 [rotary_dim / 2].  Block b = positions [b * ratio, (b + 1) * ratio): its key is the
 * mean of its raw keys, RMS-normed, rotated at position b * ratio; score(r, b) = sum over heads of
 * max(qn[r, h] . key_b, 0) / sqrt(d) for the (base_pos + r + 1) / ratio complete blocks row r sees
 * (scores f32 [rows, max_blocks]; other entries are left alone).  qw_op_qsa_pool stores the keys of
 * blocks [b0, b1) into pool f32 [max_blocks, d]; qw_op_qsa_scores_pooled scores from them, with
 * results identical to qw_op_qsa_scores.  d: a multiple of 32 from 64 to 256; rotary_dim 64. */
void qw_op_qsa_scores(qw_cmd c, qw_ref scores, qw_ref qn, qw_ref ikeys, qw_ref k_norm,
                      qw_ref inv_freq, int32_t rows, int32_t nq, int32_t d, int32_t ratio,
                      int32_t base_pos, int32_t rotary_dim, int32_t max_blocks, float eps);
void qw_op_qsa_pool(qw_cmd c, qw_ref pool, qw_ref ikeys, qw_ref k_norm, qw_ref inv_freq,
                    int32_t d, int32_t ratio, int32_t b0, int32_t b1, int32_t rotary_dim, float eps);
void qw_op_qsa_scores_pooled(qw_cmd c, qw_ref scores, qw_ref qn, qw_ref pool, int32_t rows,
                             int32_t nq, int32_t d, int32_t ratio, int32_t base_pos, int32_t max_blocks);
/* qwasar_gpu.h:635-641 -- per row the block_topk best complete blocks (one at a time: the largest
 * score above -FLT_MAX, the lowest index among equals) plus the incomplete trailing block, as a
 * byte mask (uint8 [rows, max_ctx]; positions [0, base_pos + r] of row r are written) and as the
 * list qw_op_attn_masked walks (uint32 [rows, 1 + block_topk * ratio + ratio]: count, then the
 * visible positions ascending). */
void qw_op_qsa_select(qw_cmd c, qw_ref mask, qw_ref list, qw_ref scores, int32_t rows, int32_t ratio,
                      int32_t base_pos, int32_t block_topk, int32_t max_ctx, int32_t max_blocks);
/* qwasar_gpu.h:439-446.  What the graph calls: rows >= 16 -> the tiled
 * kernel; fewer -> the split-KV kernel; the per-query kernel where those
 * decline. */
void qw_op_attn(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache,
                int32_t rows, int32_t q_heads, int32_t kv_heads,
                int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale);

/* ======================================================================== *
 *  Part 2 -- additive entry points (no counterpart in the reference)        *
 * ======================================================================== */

typedef enum { QW_F32 = 0, QW_BF16 = 1 } qw_dtype;

/* Last error of a call that has no qw_cmd to report through (allocation,
 * arena, init), or NULL. */
const char *qw_gpu_last_error(void);
int32_t     qw_gpu_sm_count(void);

/* ---- several GPUs in one process -------------------------------------------
 * qw_gpu_init brings up the calling thread's current CUDA device.  qw_gpu_init_multi brings up
 * devices 0 .. n_dev-1 and lets each read and write the others' memory (needed by the exchange of
 * partials below); device 0 is current afterwards.  qw_gpu_select makes a device current for the
 * calls that allocate (qw_buf_*, qw_kv_*, qw_xchg_create, qw_cmd_begin); a command buffer stays on
 * the device it was begun on, and ops encoded on it switch to that device by themselves, so a host
 * thread drives several GPUs by alternating between their command buffers.  Like the reference's
 * backend state (qwasar_metal.m:24-33) all of this is process-global and unsynchronised: one
 * thread at a time. */
int32_t     qw_gpu_device_count(void);
bool        qw_gpu_init_multi(int32_t n_dev, char *err, size_t errcap);
bool        qw_gpu_select(int32_t dev);
int32_t     qw_gpu_current(void);            /* -1 before init */

/* Kernels this library has launched since qw_gpu_init (every __global__ launch counts one). */
uint64_t    qw_gpu_launch_count(void);
/* Diagnostic knobs (the counterpart of the reference's QWASAR_ATTN / QWASAR_FA overrides,
 * qwasar_metal.m:1513-1516): "split_kg" = 4 | 6, consumer warps per 16-row tile of the
 * split-KV kernel (one row tile: a decode step); "split_kg2" = 3 | 2, the same for two row tiles (17 to 32 query rows
 * per KV head: a verify step); "prefill_tc" = 1 | 0, many-row attention on the tcgen05 kernel or on the
 * split-KV kernel over row chunks; "prefill_fuse_q" = 1 | 0, with bf16 rows the tcgen05 prefill norms and
 * rotates its own query tiles (default) or the pre-op kernel does; "pdl" = 1 | 0, the kernels of the
 * decode chain, of the QSA ops, of the small unfused ops and of the few-token 4-bit product start under the kernel in
 * front of them (programmatic dependent launch, default: each waits for that kernel before it touches memory) or in
 * plain stream order; "masked_tc" = 1 | 2 | 0, attention over a gathered row list on tensor-op tiles
 * (bf16 operands) as one launch on a thread-block cluster (default), as partials plus a merge launch, or on
 * the fp32 kernel; "qmv_tc" = 1 | 0, the 4-bit product of up to 15 tokens
 * on the integer tensor path (default; four tokens to a pass over the weights) or on the fp32 kernel; "qmv_pre" = 1 | 0 | 2, the
 * integer path's digits of x are cut once by a kernel ahead of the product from three tokens on (default), never
 * (every block of the product cuts its own), or for one and two tokens as well; "qmm_tc" = 1 | 0, the product for
 * 16 tokens and more (groups of 64, k a multiple of 512 from 2048 up) on the tcgen05 GEMM with fp16 operands (default;
 * the reference's tensor form and its 5e-5 bound) or on the fp32 kernel.  Returns false for an unknown
 * knob or value. */
bool        qw_gpu_tune(const char *knob, int32_t value);
/* How the split-KV decode kernel divides a launch of n_seq sequences (n_keys[i] keys each, kv_heads
 * heads) over at most n_cta_max CTAs: all (sequence, kv head) groups are laid end to end as one line
 * of 32-key tiles and share_first[c] is the first tile of CTA c's share, share_first[n] the total
 * (n = the return value = CTAs used, <= 256; share_first holds n_cta_max + 1 entries).  Shares are
 * equal in cost, a group start counting as three tiles.  *needs_merge (may be NULL) tells whether any
 * group is cut over several CTAs.  Host arithmetic only -- works without a device; 0 on bad arguments. */
int32_t     qw_attn_split_plan(int32_t n_seq, int32_t kv_heads, const int32_t *n_keys, int32_t n_cta_max,
                               int32_t *share_first, int32_t *needs_merge);
/* Per-kernel device timing for roofline figures: while on, every launch of an attention
 * kernel ("qw_attn_split", "qw_attn_prefill", "qw_attn_preop") is bracketed by a pair of CUDA events on its
 * stream; qw_cmd_wait folds the elapsed times into per-kernel totals that
 * qw_prof_kernel_read returns (false for an unknown name). */
void        qw_prof_kernels(bool on);
bool        qw_prof_kernel_read(const char *kernel, double *ms_total, int64_t *launches, bool reset);

/* Device-only buffers: no host mirror, qw_buf_contents returns NULL. */
qw_buf qw_buf_alloc_device(size_t len);                /* zero-filled */
qw_buf qw_buf_wrap_device(void *device_ptr, size_t len); /* caller keeps ownership */
void  *qw_buf_device_ptr(qw_buf b);
/* Blocking copies between host memory and any buffer's device side. */
bool   qw_buf_upload(qw_buf b, size_t off, const void *src, size_t len);
bool   qw_buf_download(qw_buf b, size_t off, void *dst, size_t len);

/* A command buffer on a stream the caller owns (a cudaStream_t passed as
 * void*), so that ops order with the caller's other work on that stream. */
qw_cmd qw_cmd_begin_on_stream(void *cuda_stream);
/* dst[0:n] = src[0:n] bytes, in stream order; either side may be a shared,
 * device or wrapped buffer. */
void   qw_op_copy(qw_cmd c, qw_ref dst, qw_ref src, size_t n);

/* ---- the paged K/V arena -------------------------------------------------
 * One arena replaces one of the reference's cache buffers (kcache or vcache:
 * [n_layers, kv_heads, max_ctx, head_dim], qwasar_graph.c:79-86).  Storage is
 * a pool of 32 KB pages (64 tokens x 256 dims x bf16, rows 512 B, so every row
 * is 128 B-aligned) mapped on demand; a device page table per (layer, head)
 * gives logical page -> pool page.  The arena's *logical* contents are those
 * of the head-major array, bit for bit, and callers keep addressing it with
 * the reference's byte offsets (layer stride kv_heads*max_ctx*head_dim*2).
 * Physical memory is committed as tokens are appended (growth in 64 MB steps
 * of a reserved virtual range), which is what the reference gets from lazily
 * committed shared buffers.  shuffle_seed != 0 hands pages out in a permuted
 * order (tests use it so that the mapping is never the identity). */
qw_buf  qw_kv_arena_alloc(int32_t n_layers, int32_t kv_heads, int32_t max_ctx, int32_t head_dim);
qw_buf  qw_kv_arena_alloc_ex(int32_t n_layers, int32_t kv_heads, int32_t max_ctx, int32_t head_dim,
                             uint32_t shuffle_seed);
/* A page pool that several arenas share: max_bytes of device addresses are reserved, memory is
 * committed as the arenas' tokens arrive.  This is the layout for serving many sequences on one
 * GPU -- one pool per GPU, one K and one V arena per sequence inside it: pages go where the
 * tokens are, and because arenas of one pool share its tensor maps, one attention launch carries
 * all their sequences (a launch holds at most 8 distinct maps; an arena from qw_kv_arena_alloc has
 * a private pool and so a map of its own).  Freeing an arena returns its pages to the pool; the
 * pool's memory goes when the pool handle and every arena in it have been freed. */
qw_buf  qw_kv_pool_alloc(size_t max_bytes, uint32_t shuffle_seed);
qw_buf  qw_kv_arena_alloc_in(qw_buf pool, int32_t n_layers, int32_t kv_heads, int32_t max_ctx, int32_t head_dim);
int64_t qw_kv_pool_bytes_committed(qw_buf pool);
/* Gather / scatter of n token rows of one (layer, head) starting at pos0,
 * to / from packed host memory (n * head_dim * 2 bytes) -- what
 * qw_session_pack / qw_session_unpack (qwasar_graph.c:320-393) need in place
 * of memcpy through qw_buf_contents.  Blocking.  Also accept a plain cache
 * buffer, for which they are strided copies. */
bool    qw_kv_read(qw_buf cache, int32_t layer, int32_t head, int32_t pos0, int32_t n, void *dst,
                   int32_t kv_heads, int32_t max_ctx, int32_t head_dim);
bool    qw_kv_store(qw_buf cache, int32_t layer, int32_t head, int32_t pos0, int32_t n, const void *src,
                    int32_t kv_heads, int32_t max_ctx, int32_t head_dim);
/* The whole KV section of the reference's packed session state in one call
 * (qw_session_pack / qw_session_unpack, qwasar_graph.c:296-303, 320-373):
 * for every layer, for every kv head, the K rows of positions [0, n_tokens)
 * then the V rows, head_dim bf16 each, nothing else.  qw_kv_state_bytes is
 * that section's size; pack wants cap >= it, unpack wants len == it (the
 * reference's own length check, qwasar_graph.c:361-362) and maps the pages it
 * fills.  Blocking; one gather or scatter kernel and one copy per layer.  The
 * element type is bf16, not the reference's IEEE half: a checkpoint written
 * by the other build must be refused by the file header, which is the
 * caller's (qwasar_kvstore.c:52-63 records no dtype yet). */
size_t  qw_kv_state_bytes(int32_t n_layers, int32_t kv_heads, int32_t head_dim, int32_t n_tokens);
/* What a checkpoint header should record beside its dims so that a payload written by a build with
 * another cache element type is rejected rather than misread: the four characters "BF16" as a
 * little-endian word (0x36314642).  The reference's header (qwasar_kvstore.c:52-63) has a `reserved`
 * word for it; a build that stores IEEE half would write "F16 ". */
uint32_t qw_kv_element_tag(void);
bool    qw_kv_pack(qw_buf kcache, qw_buf vcache, int32_t n_layers, int32_t kv_heads, int32_t max_ctx,
                   int32_t head_dim, int32_t n_tokens, void *dst, size_t cap);
bool    qw_kv_unpack(qw_buf kcache, qw_buf vcache, int32_t n_layers, int32_t kv_heads, int32_t max_ctx,
                     int32_t head_dim, int32_t n_tokens, const void *src, size_t len);
/* Returns to the pool every page that lies wholly at or past n_tokens
 * (a rewind, qwasar_graph.c:407-463, needs no undo of KV rows; this only
 * gives memory back). */
void    qw_kv_arena_trim(qw_buf cache, int32_t n_tokens);
int64_t qw_kv_arena_pages_in_use(qw_buf cache);
int64_t qw_kv_arena_bytes_committed(qw_buf cache);

/* ---- the fused node ------------------------------------------------------
 * Everything qw_encode_attention_layer encodes between the q/k/v projections
 * and o_proj (qwasar_graph.c:630-659), in two or three launches: split of
 * [q|gate], RMS norm of q and k (bf16 weights or null refs), partial RoPE,
 * K/V append at base_pos, causal attention of the rows against
 * [0, base_pos + r], sigmoid output gate.
 *   qg   [rows, q_heads, 2*head_dim]   k, v  [rows, kv_heads, head_dim]   (io)
 *   out  [rows, q_heads, head_dim]                                        (io)
 * io = QW_F32 or QW_BF16 for qg, k, v and out alike.  Returns false, encoding
 * nothing, for head_dim != 256, rotary_dim != 64 or q_heads % kv_heads != 0. */
bool qw_op_attn_layer_fused(qw_cmd c, qw_ref out, qw_ref qg, qw_ref k, qw_ref v,
                            qw_ref q_norm_w, qw_ref k_norm_w, qw_ref pos, qw_ref axis, qw_ref inv_freq,
                            qw_ref kcache, qw_ref vcache, int32_t rows, int32_t q_heads, int32_t kv_heads,
                            int32_t head_dim, int32_t rotary_dim, int32_t max_ctx, int32_t base_pos,
                            float eps, float scale, qw_dtype io);

/* The same for n_seq independent sequences (one qw_session each in the
 * reference, which has no batch dimension): arrays of n_seq refs and base
 * positions; every sequence has `rows` rows.  One launch of each kernel carries
 * up to 64 sequences whose caches lie in at most 8 distinct buffers or pools
 * (arenas of one pool count once); more are taken in further launches. */
bool qw_op_attn_layer_fused_batch(qw_cmd c, int32_t n_seq, const qw_ref *out, const qw_ref *qg,
                                  const qw_ref *k, const qw_ref *v, qw_ref q_norm_w, qw_ref k_norm_w,
                                  const qw_ref *pos, qw_ref axis, qw_ref inv_freq,
                                  const qw_ref *kcache, const qw_ref *vcache, const int32_t *base_pos,
                                  int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                                  int32_t rotary_dim, int32_t max_ctx, float eps, float scale, qw_dtype io);

/* Batched form of qw_op_attn (attention only; q/out fp32 or bf16 per `io`). */
bool qw_op_attn_batch(qw_cmd c, int32_t n_seq, const qw_ref *out, const qw_ref *q,
                      const qw_ref *kcache, const qw_ref *vcache, const int32_t *base_pos,
                      int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                      int32_t max_ctx, float scale, qw_dtype io);

/* ---- partials, for a sequence split across GPUs ---------------------------
 * qw_op_attn_partial attends the rows to the cache positions
 * [key_lo, key_hi) only (key_lo a multiple of 64; causality still applies) and
 * leaves, per (row, query head), the un-normalised partial softmax:
 *   pacc  f32 [rows, q_heads, head_dim]   sum_t exp(s_t - m) V_t
 *   pstat f32 [rows, q_heads, 2]          (m, sum_t exp(s_t - m)); sum 0 = no keys
 * -- the (max, sum, acc) triple of the reference's split kernels
 * (metal/attn.metal:198-259).  qw_op_attn_merge combines `parts` such sets,
 * laid out [parts, rows*q_heads, ...] (what an all-gather of the ranks'
 * partials produces), by log-sum-exp exactly as qw_attn_merge_gated does
 * (metal/attn.metal:273-331), applying sigmoid(gate) when gate is not a null
 * ref; gate element (r, h, d) is read at gate[(r*q_heads + h)*gate_stride + d].
 * part_stride: floats between consecutive parts in both pacc and pstat, for partials that
 * were gathered as one packed record per rank (acc block then stat block); 0 = the dense
 * layouts above. */
bool qw_op_attn_partial(qw_cmd c, qw_ref pacc, qw_ref pstat, qw_ref q, qw_ref kcache, qw_ref vcache,
                        int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                        int32_t max_ctx, int32_t base_pos, int32_t key_lo, int32_t key_hi,
                        float scale, qw_dtype q_dtype);
void qw_op_attn_merge(qw_cmd c, qw_ref out, qw_ref pacc, qw_ref pstat, qw_ref gate,
                      int32_t rows, int32_t q_heads, int32_t head_dim, int32_t parts,
                      int32_t gate_stride, qw_dtype out_dtype, qw_dtype gate_dtype, int64_t part_stride);

/* ---- the exchange of partials between GPUs ---------------------------------
 * For a sequence whose positions are split over n_ranks GPUs (2 to 8; one process per GPU, or one
 * process that holds them all).  Each rank creates one qw_xchg on its device: a gather buffer with
 * a slot and a flag per (rank, row, head) for rows * q_heads <= max_rows_heads.  The ranks swap
 * handles once -- qw_xchg_export writes qw_xchg_handle_bytes() (64) bytes to pass to the other
 * processes by any means, qw_xchg_attach maps a peer's buffer from its handle (CUDA IPC),
 * qw_xchg_attach_local takes the peer's object directly when it lives in this process (after
 * qw_gpu_init_multi).  After that no library call and no host synchronisation is involved:
 * qw_op_attn_exchange attends this rank's rows to its own key range [key_lo, key_hi) like
 * qw_op_attn_partial, then its combine kernel stores the (acc, max, sum) record of every (row,
 * head) straight into every rank's gather buffer (peer stores over NVLink) and raises the flags
 * beside them, waits until the flags of all ranks are in, merges by log-sum-exp, applies the gate
 * and writes out -- on every rank the full result (metal/attn.metal:273-331 is the arithmetic; the
 * exchange itself is new).  Two kernels per call.  phase 0 does all of it; phase 1 stops after
 * publishing and phase 2 only waits, merges and writes (1 then 2 equals 0: for hosts that want
 * other work between the halves, and the only form in which several ranks may share ONE GPU,
 * where a kernel must never wait for a kernel launched after it).
 * Every rank must make the same sequence of calls on its exchange.  The wait is bounded
 * (qw_xchg_set_timeout_ms, default 2000): a rank whose peers' records do not arrive gives up,
 * writes no output, and qw_cmd_error reports it after qw_cmd_wait. */
typedef struct qw_xchg_s *qw_xchg;
qw_xchg qw_xchg_create(int32_t n_ranks, int32_t rank, int32_t max_rows_heads);
void    qw_xchg_free(qw_xchg x);
size_t  qw_xchg_handle_bytes(void);
bool    qw_xchg_export(qw_xchg x, void *handle);
bool    qw_xchg_attach(qw_xchg x, int32_t peer_rank, const void *handle);
bool    qw_xchg_attach_local(qw_xchg x, int32_t peer_rank, qw_xchg peer);
void    qw_xchg_set_timeout_ms(qw_xchg x, int32_t ms);
bool    qw_op_attn_exchange(qw_cmd c, qw_xchg x, int32_t phase, qw_ref out, qw_ref gate, qw_ref q,
                            qw_ref kcache, qw_ref vcache, int32_t rows, int32_t q_heads, int32_t kv_heads,
                            int32_t head_dim, int32_t max_ctx, int32_t base_pos, int32_t key_lo, int32_t key_hi,
                            float scale, qw_dtype q_dtype, qw_dtype out_dtype, qw_dtype gate_dtype,
                            int32_t gate_stride);
/* The same round for n_seq (<= 64) sequences of equal shape in the same two kernels: arrays of
 * n_seq refs, positions and key ranges; gate may be NULL; n_seq * rows * q_heads <= max_rows_heads. */
bool    qw_op_attn_exchange_batch(qw_cmd c, qw_xchg x, int32_t phase, int32_t n_seq, const qw_ref *out,
                                  const qw_ref *gate, const qw_ref *q, const qw_ref *kcache, const qw_ref *vcache,
                                  const int32_t *base_pos, const int32_t *key_lo, const int32_t *key_hi,
                                  int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_ctx,
                                  float scale, qw_dtype q_dtype, qw_dtype out_dtype, qw_dtype gate_dtype,
                                  int32_t gate_stride);

/* The pre-op half of the fused node alone (split, norm, RoPE, append; q_out
 * receives the normed + roped query as bf16 [rows, q_heads, head_dim]), for
 * callers that run the attention half per rank (sequence split). */
bool qw_op_attn_preop(qw_cmd c, qw_ref q_out, qw_ref qg, qw_ref k, qw_ref v,
                      qw_ref q_norm_w, qw_ref k_norm_w, qw_ref pos, qw_ref axis, qw_ref inv_freq,
                      qw_ref kcache, qw_ref vcache, int32_t rows, int32_t q_heads, int32_t kv_heads,
                      int32_t head_dim, int32_t rotary_dim, int32_t max_ctx, int32_t base_pos,
                      float eps, qw_dtype io, bool append);

/* ---- decode attention without any allocation --------------------------------
 * No counterpart in the reference, whose buffers all come from its own
 * allocator (qw_buf_alloc / qw_cmd_scratch).
 *
 * For callers that cannot let this library allocate: an embedder that gave all
 * device memory to its own pool at start-up, or a serving loop in a phase where
 * cudaMalloc is forbidden because it stalls every stream of the device.  The
 * ordinary attention ops draw their partial-softmax scratch from a pool that
 * grows by cudaMalloc on first use; this entry point instead keeps its scratch
 * in a fixed array inside the library image (qw_attn_decode_noalloc_scratch_bytes()
 * = 4 MiB, resident on every GPU that loads the library until the process ends)
 * and calls no cudaMalloc, cudaFree or other allocating routine.  It does not
 * need qw_gpu_init either.
 *
 * Split-KV attention of `rows` query rows (the new token, or a few speculative
 * ones) of one sequence against a head-major cache, same arithmetic and result
 * as qw_op_attn_decode_tensor, optionally with the sigmoid output gate.  All
 * pointers are device pointers the caller owns:
 *   out, q   [rows, q_heads, 256]   gate: the same shape, or NULL   (f32 or bf16 per `io`)
 *   kcache, vcache   bf16 [kv_heads, max_ctx, 256], 128-byte aligned
 *   cuda_stream      a cudaStream_t (NULL = the default stream)
 * Limits: head_dim 256; rows * (q_heads / kv_heads) <= 16; the scratch this
 * shape needs, (SMs + kv_heads) * 16 + rows * q_heads partial rows of 1032
 * bytes, must fit the array -- otherwise false is returned with the reason in
 * err, and nothing is launched.
 *
 * The first call on each device (made with that device current) resolves the
 * array's device address and sets a kernel attribute; make that call before
 * any stream capture begins, and from one thread: that first-call set-up is not
 * guarded against two threads entering it at once.  The call returns when its
 * kernels are queued.  A kernel whose bounded internal wait runs out (a fault
 * of the device, not of the arguments) cannot be reported through the return
 * value: after synchronising, qw_attn_decode_noalloc_status() returns, and
 * clears, the code it left (0 = none; the output of such a call is not valid).
 * All calls on a device share the one array: two
 * calls whose kernels overlap on the GPU (different streams, no dependency)
 * race on it -- order them on one stream or with events.  Nothing in the array
 * needs clearing between calls; stale contents are never read. */
bool   qw_attn_decode_noalloc(void *out, const void *q, const void *gate, const void *kcache, const void *vcache,
                              int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                              int32_t max_ctx, int32_t base_pos, float scale, qw_dtype io, void *cuda_stream,
                              char *err, size_t errcap);
size_t qw_attn_decode_noalloc_scratch_bytes(void);
int32_t qw_attn_decode_noalloc_status(void);

#ifdef __cplusplus
}
#endif
#endif /* QWASAR_CUDA_H */
