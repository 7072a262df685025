// Internal launch interface between the C-ABI backend (qwasar_cuda.cu) and the
// kernel translation units.  Not part of the public boundary.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include "qw_common.cuh"

namespace qw {

enum Dtype : int { DT_F32 = 0, DT_BF16 = 1 };

// Where one layer's K (or V) rows live.  Row index `row(h, t)` addresses a 512-byte
// row of a 2-D [total_rows, 256] bf16 array:
//   linear (reference layout, qwasar_gpu.h:395-400): row = h * max_ctx + t
//   paged  (arena):  row = table[h * pt_stride + t / 64] * 64 + t % 64
struct KvLayer {
    __nv_bfloat16 *base;     // row 0 of the 2-D array (linear: the layer's first row; paged: the pool)
    const int32_t *table;    // paged: this layer's page table [kv_heads, pt_stride]; linear: nullptr
    int32_t pt_stride;
    int32_t max_ctx;
};

__host__ __device__ __forceinline__ int64_t kv_row(const KvLayer &L, int32_t h, int32_t t) {
#ifdef __CUDA_ARCH__
    if (L.table) return (int64_t)__ldg(L.table + (size_t)h * L.pt_stride + (t >> 6)) * QW_PAGE_TOKENS + (t & 63);
#endif
    return (int64_t)h * L.max_ctx + t;
}

// ---- pre-ops -------------------------------------------------------------------------
void launch_split_heads2(cudaStream_t s, float *a, float *b, const float *src, int rows, int heads, int dim);
void launch_rms_norm(cudaStream_t s, float *y, const float *x, const uint16_t *w, int dim, int rows, float eps,
                     float out_scale);
void launch_rope_partial(cudaStream_t s, float *x, const int32_t *pos, const uint8_t *axis, const float *inv_freq,
                         int rows, int heads, int head_dim, int rotary_dim);
void launch_kv_write(cudaStream_t s, KvLayer kc, KvLayer vc, const float *k, const float *v, int rows, int kv_heads,
                     int base_pos);
void launch_mul_sigmoid(cudaStream_t s, float *y, const float *gate, int64_t n);
// One layer between the cache and the packed layout [kv_heads][K rows | V rows][n_tokens][256] bf16.
void launch_kv_pack(cudaStream_t s, KvLayer kc, KvLayer vc, void *packed, int kv_heads, int n_tokens, bool unpack);
void launch_f32_to_bf16(cudaStream_t s, __nv_bfloat16 *dst, const float *src, int64_t n);
void launch_slice_rows(cudaStream_t s, float *dst, const float *src, int rows, int src_stride, int offset, int len);

// One sequence of the fused pre-op: split [q|gate], RMS-norm q and k, partial RoPE,
// round and append K/V, leave the normed+roped query as bf16.
struct PreopSeq {
    const void *qg;          // [rows, q_heads, 512]   (io dtype)
    const void *k, *v;       // [rows, kv_heads, 256]  (io dtype)
    const int32_t *pos;      // [3, rows]
    __nv_bfloat16 *q_out;    // [rows, q_heads, 256]
    float *cs_out;           // nullptr, or [rows, 64]: cos then sin of the 32 rotation angles of every row
    KvLayer kc, vc;
    int32_t rows, base_pos;
};
struct PreopParams {
    PreopSeq seq[QW_MAX_SEQ];
    int32_t n_seq, q_heads, kv_heads, rotary_dim, io_dtype;
    int32_t skip_q;                        // leave the query heads alone (the prefill kernel norms and rotates its own tiles)
    const uint16_t *q_norm_w, *k_norm_w;   // bf16 [256] or nullptr
    const uint8_t *axis;
    const float *inv_freq;
    float eps;
};
void launch_preop(cudaStream_t s, const PreopParams &p, int max_rows);

// ---- attention ------------------------------------------------------------------------
struct AttnSeq {
    const void *q;           // [rows, q_heads, 256] f32 or bf16; with q_raw the [q|gate] rows [rows, q_heads, 512]
    void *out;               // [rows, q_heads, 256] f32 or bf16
    const void *gate;        // nullptr, or element (r, h, d) at gate[(r*q_heads + h)*gate_stride + d]
    const int32_t *pos;      // q_raw: positions of this sequence's first row, axis a of row r at pos[a*pos_stride + r]
    KvLayer kc, vc;
    int32_t rows, base_pos;  // row r reads keys [key_lo, min(key_hi, base_pos + r + 1))
    int32_t key_lo, key_hi;  // this launch's share of the sequence (whole: 0, base_pos + rows)
    int32_t tile0, n_tiles;  // first 32-key tile and tile count per kv head, from key_lo/key_hi
    int32_t cum_tiles;       // tiles of all earlier sequences times kv_heads
    int32_t row_slot0;       // first row of this sequence in the partial buffers
    int32_t pos_stride;      // q_raw: rows of the call the positions belong to
    int32_t fresh_pos;       // early: first cache position the kernel in front of this launch appends
    uint8_t kmap, vmap;      // which of the launch's tensor maps cover this sequence's K and V rows
};
// Partials that cross GPUs (a sequence split by position): every rank stores its combined
// (acc, max, sum) record of each (row, head) straight into every rank's gather buffer and raises
// a flag beside it; a rank merges once the flags of all ranks are in.
struct XchgDev {
    float *gather[8];        // rank i's buffer [2 parities][n_ranks][max_rh][258] (acc[256], max, sum), as seen from this GPU
    int *flags[8];           // rank i's flags  [2 parities][n_ranks][max_rh]: the epoch of the record beside it
    int32_t n_ranks, rank, max_rh, epoch;
    int32_t empty;           // no sequence of this launch has a visible key in this rank's range: empty records go out
    int64_t timeout_ns;      // how long a rank waits for the others' records before it reports QW_ST_PEER_TIMEOUT
};
struct AttnParams {
    CUtensorMap maps[QW_MAX_MAPS];
    AttnSeq seq[QW_MAX_SEQ];
    int32_t n_seq, q_heads, kv_heads, gqa;
    int32_t q_dtype, out_dtype, gate_dtype, gate_stride;
    int32_t total_tiles, n_cta;
    // 0: write normalised (gated) output; 1: leave one combined partial (m, l, acc) per (row, head);
    // 2: publish that partial to all ranks of an exchange, wait for theirs, merge and write the output;
    // 3: publish only; 4: wait + merge + output only (3 then 4 is 2 in two launches)
    int32_t mode;
    // q_raw: the kernel applies the per-head RMS norm (weights q_norm_w, bf16 [256] or nullptr) and the
    // partial RoPE (axis uint8 [32], inv_freq f32 [32]) to the raw query rows itself
    int32_t q_raw;
    // early: launched directly behind this node's own K/V append kernel; only the tiles from each
    // sequence's fresh_pos on wait for it (see pdl_wait in qw_common.cuh)
    int32_t early;
    const uint16_t *q_norm_w;
    const uint8_t *axis;
    const float *inv_freq;
    float eps;
    float scale;
    float *pacc, *pstat;     // partial scratch: [slot, MT*16, 256] and [slot, MT*16, 2]
    float *comb_acc, *comb_stat;   // mode 1: where the one combined partial per (row, head) goes
    int *status;
    XchgDev x;               // modes 2-4
};
// rows_per_seq * gqa <= 64.  The number of partial slots a launch may write: a (CTA, group)
// segment uses slot cta + group.
__host__ __device__ inline int attn_split_slots(const AttnParams &p) { return p.n_cta + p.n_seq * p.kv_heads; }
size_t attn_split_scratch_bytes(const AttnParams &p, int max_rows);
void launch_attn_split(cudaStream_t s, const AttnParams &p, int max_rows);
void launch_attn_merge(cudaStream_t s, const AttnParams &p, int max_rows);
bool attn_split_needs_merge(const AttnParams &p);
void attn_split_shares(const AttnParams &p, int32_t *share_first);

// Causal prefill on tcgen05 tensor cores: one CTA per (128-row tile, query head).
struct PrefillParams {
    const __nv_bfloat16 *q;  // [rows, q_heads, 256], 16-byte aligned
    CUtensorMap kmap, vmap;  // cache row maps, box 64 x 64
    // Tile maps of the single-CTA kernel, all SWIZZLE_128B with 128-byte x 128-row boxes: q as
    // [rows][q_heads*256] bf16; out the same shape in out_dtype; gate as [rows][q_heads*gate_stride]
    // in gate_dtype (== out_dtype).  Bases 16-byte aligned, row pitches multiples of 16 bytes.
    CUtensorMap qmap, omap, gmap;
    // fuse_q: qmap covers the raw [q|gate] rows ([rows][q_heads*512] bf16) and the kernel applies the
    // per-head RMS norm (weights q_norm_w, bf16 [256] or nullptr) and the partial RoPE itself, with the
    // angles' cos / sin read from csmap ([rows][64] f32, written by the pre-op's key warps).
    CUtensorMap csmap;
    const uint16_t *q_norm_w;
    float eps;
    int32_t fuse_q;
    KvLayer kc, vc;
    void *out;               // [rows, q_heads, 256] f32 or bf16
    const void *gate;        // nullptr or element (r, h, d) at gate[(r*q_heads + h)*gate_stride + d]
    int32_t out_dtype, gate_dtype, gate_stride;
    int32_t rows, base_pos, q_heads, kv_heads, gqa, n_q_tiles;
    int32_t oob_row;         // a row index past both cache maps: TMA fills zeros there
    float scale;
    int *status;
};
void launch_attn_prefill(cudaStream_t s, const PrefillParams &p);
// Whether out / gate can be described by the tile maps above (alignment, equal dtypes).
bool attn_prefill_io_ok(const void *out, int out_dtype, const void *gate, int gate_dtype, int gate_stride);

// Per-query fp32 kernel (CUDA cores, no rounding of q or of the weights).
// list != nullptr: row r attends only the positions list[r * list_stride + 1 ...] (count at [0]).
void launch_attn_per_query(cudaStream_t s, const AttnSeq &seq, int q_heads, int kv_heads, float scale,
                           float *pacc, float *pstat, int splits, const uint32_t *list = nullptr, int list_stride = 0);
size_t attn_per_query_scratch_bytes(int rows, int q_heads, int splits);
int attn_per_query_splits(int rows, int q_heads, int n_keys);

// Masked attention on tensor ops over each row's position list (q f32; grouping <= 16): one partial
// per 64 list entries into pacc [chunks, rows * q_heads, 256] / pstat [chunks, rows * q_heads, 2].
int attn_masked_chunks(int cap);
bool launch_attn_masked_cluster(cudaStream_t s, const AttnSeq &seq, int q_heads, int kv_heads, float scale, const uint32_t *list,
                                int list_stride, float *out, const float *gate, int gate_stride);
void launch_attn_masked_mma(cudaStream_t s, const AttnSeq &seq, int q_heads, int kv_heads, float scale, const uint32_t *list,
                            int list_stride, float *pacc, float *pstat);

// Merge of externally supplied partials (the cross-GPU exchange): pacc [parts, rows*q_heads, 256],
// pstat [parts, rows*q_heads, 2] -> out (gated when gate != nullptr).
void launch_merge_parts(cudaStream_t s, void *out, int out_dtype, const float *pacc, const float *pstat,
                        const void *gate, int gate_dtype, int gate_stride, int n_rows_heads, int parts,
                        float *pacc_out, float *pstat_out, size_t acc_stride = 0, size_t stat_stride = 0);

// ---- 4-bit affine product (qw_qmat.cu): y [rows, n] = x [rows, k] . dequant(w [n, k/8])^T ----
// `xq`: qmv_scratch_bytes(rows, k, group) bytes of scratch for the digits of x (0: none wanted), or null (the kernel's blocks
// then cut the digits themselves).
size_t qmv_scratch_bytes(int rows, int k, int group);
void launch_qmat_q4(cudaStream_t s, float *y, const float *x, const uint32_t *w, const uint16_t *scales, const uint16_t *biases, int k,
                    int n, int rows, int group, int *status, void *xq);

// Up to four one-token products sharing x (and k, group) in one launch; w rows 16-byte aligned.
struct QmvMulti {
    float *y[4];
    const uint32_t *w[4];
    const uint16_t *scales[4], *biases[4];
    const float *x;
    int32_t n[4], blocks[4];
    int32_t count, k, group;
};
void launch_qmv_q4_multi(cudaStream_t s, QmvMulti m, int *status, void *xq);

// ---- the 4-bit product for many tokens on tcgen05 (qw_qgemm.cu) --------------------------------
struct QgemmParams {
    CUtensorMap map_x;       // fp16 [rows, k] (elements of every 8 in the order 0 4 1 5 2 6 3 7), boxes 64 x 128, SWIZZLE_128B
    CUtensorMap map_w;       // u32 [n, k / 8], boxes 8 x 256
    CUtensorMap map_s, map_b;  // bf16 [n, k / 64], boxes 8 x 256
    float *y;                // [rows, n]
    int *status;
    int32_t rows, n, k;
    int32_t halves;          // 128-token halves per tile (set by the launcher)
    int32_t split_from;      // tiles from this one on run as two entries of one half each (set by the launcher)
};
size_t qgemm_scratch_bytes(int rows, int k);
bool launch_qgemm_q4(cudaStream_t s, const QgemmParams &p, const float *x, void *x16);
extern int g_tune_qmm_tc;

// ---- QSA indexer (qw_qsa.cu) ----------------------------------------------------------------
void launch_qsa_pool(cudaStream_t s, float *pool, const float *ikeys, const uint16_t *k_norm, const float *inv_freq, int d, int ratio,
                     int b0, int b1, float eps);
void launch_qsa_scores(cudaStream_t s, float *scores, const float *qn, const float *pool, int rows, int nq, int d, int ratio,
                       int base_pos, int max_blocks);
void launch_qsa_select(cudaStream_t s, uint8_t *mask, uint32_t *list, const float *scores, int rows, int ratio, int base_pos,
                       int block_topk, int max_ctx, int max_blocks);

int sm_count();


// Launch accounting: every launcher adds the kernels it launched.
extern unsigned long long g_launches;
// Key groups (consumer warps per 16-row tile) of the split-KV kernel at one row tile: 4 or 6.
extern int g_tune_split_kg;
// 1: many-row attention runs on the tcgen05 kernel; 0: on the split-KV kernel over row chunks.
extern int g_tune_prefill_tc;
// 1: with bf16 rows the tcgen05 prefill norms and rotates its own query tiles; 0: the pre-op does.
extern int g_tune_prefill_fuse_q;
// 1: the kernels of the decode chain are launched as programmatic dependents (they may start under
// the kernel in front of them); 0: plain stream order, for comparison.
extern int g_tune_pdl;
// 1: masked attention (position lists) on tensor ops where the grouping allows; 0: the fp32 per-query kernel.
extern int g_tune_masked_tc;
// 1: a one-token 4-bit product keeps x in registers (qmv1_q4_kernel); 0: the shared-memory kernel.
extern int g_tune_qmv_tc;
extern int g_tune_split_kg2;
extern int g_tune_qmv_pre;

}  // namespace qw
