// Pre- and post-ops of the gated attention node: head split, per-head RMS norm,
// partial RoPE, KV append, sigmoid gate -- as separate kernels behind the
// reference's op signatures, and as one fused kernel for the node.
//
// All of it is element work on 256-wide head rows, one warp per row, nothing read twice.
//
// Arithmetic follows the reference's scalar twins operation for operation
// (qwasar_cpu.c:68-82, 304-319, 344-355) with contraction switched off through
// the _rn intrinsics.  In the fused kernel the key rows -- whose bits end up in
// the cache -- also keep the twins' order of the 256-term sum of squares (left to
// right) and take cos / sin from the double-precision functions rounded once to
// float, which is what a correctly rounded cosf / sinf returns; so the appended K
// equals the CPU code's bit for bit.  Query rows (rounded to bf16 for the tensor
// cores anyway) and the stand-alone norm op sum as a tree.
#include "qw_kernels.h"

namespace qw {

namespace {

// ---- unfused ops, reference signatures ------------------------------------------------

__global__ void split_heads2_kernel(float *__restrict__ a, float *__restrict__ b, const float *__restrict__ src,
                                    int64_t n_rh, int dim) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // over n_rh * dim
    pdl_wait();                                                   // (programmatic dependent launch, qw_common.cuh)
    pdl_launch_next();
    if (i >= n_rh * dim) return;
    const int64_t rh = i / dim;
    const int d = (int)(i - rh * dim);
    a[i] = src[rh * 2 * dim + d];
    b[i] = src[rh * 2 * dim + dim + d];
}

// General RMS norm (any dim): one warp per row, strided lanes.
__global__ void rms_norm_kernel(float *__restrict__ y, const float *__restrict__ x, const uint16_t *__restrict__ w,
                                int dim, int rows, float eps, float out_scale) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_wait();                                                   // (programmatic dependent launch, qw_common.cuh)
    pdl_launch_next();
    if (row >= rows) return;
    const float *xr = x + (size_t)row * dim;
    float *yr = y + (size_t)row * dim;
    float ss = 0.0f;
    for (int i = lane; i < dim; i += 32) ss = __fadd_rn(ss, __fmul_rn(xr[i], xr[i]));
    ss = warp_sum(ss);
    const float inv = __fmul_rn(__fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)dim), eps))), out_scale);
    for (int i = lane; i < dim; i += 32) {
        float t = __fmul_rn(xr[i], inv);
        if (w) t = __fmul_rn(t, bf16_bits_to_f32(w[i]));
        yr[i] = t;
    }
}

__global__ void rope_partial_kernel(float *__restrict__ x, const int32_t *__restrict__ pos,
                                    const uint8_t *__restrict__ axis, const float *__restrict__ inv_freq,
                                    int rows, int heads, int head_dim, int half) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // over rows*heads*half
    pdl_wait();                                                   // (programmatic dependent launch, qw_common.cuh)
    pdl_launch_next();
    if (i >= (int64_t)rows * heads * half) return;
    const int j = (int)(i % half);
    const int64_t rh = i / half;
    const int r = (int)(rh / heads);
    const float ang = __fmul_rn((float)pos[(size_t)axis[j] * rows + r], inv_freq[j]);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    float *v = x + rh * head_dim;
    const float lo = v[j], hi = v[j + half];
    v[j] = __fsub_rn(__fmul_rn(lo, cs), __fmul_rn(hi, sn));
    v[j + half] = __fadd_rn(__fmul_rn(hi, cs), __fmul_rn(lo, sn));
}

// One warp per (row, kv head): 256 floats of K and of V -> bf16, 16 bytes per lane.
__global__ void kv_write_kernel(KvLayer kc, KvLayer vc, const float *__restrict__ k, const float *__restrict__ v,
                                int rows, int kv_heads, int base_pos) {
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_wait();                                                   // (programmatic dependent launch, qw_common.cuh)
    pdl_launch_next();
    if (w >= rows * kv_heads) return;
    const int r = w / kv_heads, h = w % kv_heads;
    const float4 *ks = reinterpret_cast<const float4 *>(k + (size_t)w * 256) + lane * 2;
    const float4 *vs = reinterpret_cast<const float4 *>(v + (size_t)w * 256) + lane * 2;
    const float4 k0 = ks[0], k1 = ks[1], v0 = vs[0], v1 = vs[1];
    uint4 ko, vo;
    ko.x = pack_bf16(k0.x, k0.y); ko.y = pack_bf16(k0.z, k0.w); ko.z = pack_bf16(k1.x, k1.y); ko.w = pack_bf16(k1.z, k1.w);
    vo.x = pack_bf16(v0.x, v0.y); vo.y = pack_bf16(v0.z, v0.w); vo.z = pack_bf16(v1.x, v1.y); vo.w = pack_bf16(v1.z, v1.w);
    const int64_t kr = kv_row(kc, h, base_pos + r), vr = kv_row(vc, h, base_pos + r);
    if (kr < 0 || vr < 0) return;   // unmapped page: the host maps pages before launching
    reinterpret_cast<uint4 *>(kc.base + kr * 256)[lane] = ko;
    reinterpret_cast<uint4 *>(vc.base + vr * 256)[lane] = vo;
}

__global__ void mul_sigmoid_kernel(float *__restrict__ y, const float *__restrict__ g, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_wait();                                                   // (programmatic dependent launch, qw_common.cuh)
    pdl_launch_next();
    if (i < n) y[i] = __fmul_rn(y[i], __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g[i]))));
}

// dst[r, 0:len] = src[r, offset:offset+len] over rows of src_stride floats (qwasar_gpu.h:387-389)
__global__ void slice_rows_kernel(float *__restrict__ dst, const float *__restrict__ src, int64_t n, int src_stride, int offset, int len) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_wait();                                                   // (programmatic dependent launch, qw_common.cuh)
    pdl_launch_next();
    if (i >= n) return;
    const int64_t r = i / len;
    dst[i] = src[r * src_stride + offset + (i - r * len)];
}

__global__ void f32_to_bf16_kernel(__nv_bfloat16 *__restrict__ dst, const float *__restrict__ src, int64_t n) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    pdl_wait();                                                   // (programmatic dependent launch, qw_common.cuh)
    pdl_launch_next();
    if (i + 3 < n) {
        const float4 v = *reinterpret_cast<const float4 *>(src + i);
        uint2 o;
        o.x = pack_bf16(v.x, v.y);
        o.y = pack_bf16(v.z, v.w);
        *reinterpret_cast<uint2 *>(dst + i) = o;
    } else {
        for (int64_t j = i; j < n; j++) dst[j] = __float2bfloat16_rn(src[j]);
    }
}

// ---- one layer's rows between the cache and the packed checkpoint layout ------------------
// packed: for every kv head, its K rows [n_tokens][256] then its V rows (qwasar_graph.c:296-303,
// 332-339 for one layer).  One warp per 512-byte row; a position whose page was never mapped packs
// as zeros.
__global__ void __launch_bounds__(256) kv_pack_kernel(KvLayer kc, KvLayer vc, uint4 *__restrict__ packed, int kv_heads,
                                                      int n_tokens, bool unpack) {
    const int64_t w = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= (int64_t)kv_heads * 2 * n_tokens) return;
    const int t = (int)(w % n_tokens);
    const int hv = (int)(w / n_tokens);                  // head * 2 + (0: K, 1: V)
    const int h = hv >> 1;
    const KvLayer &L = (hv & 1) ? vc : kc;
    int64_t row = -1;
    if (L.table) {
        const int32_t id = __ldg(L.table + (size_t)h * L.pt_stride + (t >> 6));
        if (id >= 0) row = (int64_t)id * QW_PAGE_TOKENS + (t & 63);
    } else {
        row = (int64_t)h * L.max_ctx + t;
    }
    uint4 *cache_row = row >= 0 ? reinterpret_cast<uint4 *>(L.base + row * 256) + lane : nullptr;
    uint4 *pk = packed + w * 32 + lane;
    if (unpack) { if (cache_row) *cache_row = *pk; }
    else *pk = cache_row ? *cache_row : make_uint4(0, 0, 0, 0);
}

// ---- the fused pre-op ---------------------------------------------------------------------
// grid = (ceil(max_rows / PRE_ROWS) * ceil(slots / PRE_WARPS), 1, n_seq) with slots = q_heads + 2 *
// kv_heads (the query heads are left out when the attention kernel norms its own rows).  A block
// covers PRE_ROWS consecutive tokens and PRE_WARPS slots, one warp per slot: slot < q_heads is a
// query head, then the key heads, then the value heads.
//
// Lane l holds the eight consecutive dims 8l .. 8l+7 of a head row: one 16-byte load and one
// 16-byte store per bf16 row and lane, no staging.  The RoPE pair (d, d + 32), d < 32, then sits
// in lanes l and l ^ 4 (l < 8) at the same register.  The 32 angles of a token are the same for
// all its heads: the block's first PRE_ROWS warps compute cos / sin once, into shared memory.
// The kernel issues few bytes per instruction, so the instruction count per row is what it pays for.
#ifndef QW_PRE_ROWS
#define QW_PRE_ROWS 4
#endif
constexpr int PRE_ROWS = QW_PRE_ROWS;
// Slots (warps) per block.  Four, not eight: the key warps live longest (their in-order sum), and a
// block holds its SM resources until its last warp is done -- with small blocks the value and query
// rows of other blocks stream under them.
constexpr int PRE_WARPS = 4;
static_assert(PRE_WARPS >= PRE_ROWS, "a block's first PRE_ROWS warps work out the rows' angles");
// cosf / sinf of an fp32 angle as the correctly rounded float (what the CPU statement gets from libm,
// qwasar_cpu.c:312-315): evaluated in double to about 2e-16 and rounded once.  The angle is reduced by
// multiples of pi / 2 in two fused steps (pi / 2 as a double and its residual; angles here stay below 2^19, so
// the product is exact to far below the result's last bit), sine and cosine of the remainder on [-pi / 4, pi / 4] are
// their Taylor sums to r^17 and r^16 (remainders below 1e-19 and 2e-18), the quadrant picks and signs them.
// About 60 instructions; the library's double sincos, which is accurate over the whole double range, cost 700 --
// two fifths of this kernel's instructions at 4096 tokens.
__device__ __forceinline__ void sincos_rounded(float ang, float &sn, float &cs) {
    const double x = (double)ang;
    const double k = rint(x * 0.63661977236758134308);
    double r = fma(-k, 1.57079632679489655800, x);
    r = fma(-k, 6.12323399573676603587e-17, r);
    const double r2 = r * r;
    double s = 1.0 / 355687428096000.0;                  // 1 / 17!
    s = fma(s, r2, -1.0 / 1307674368000.0);              // -1 / 15!
    s = fma(s, r2, 1.0 / 6227020800.0);                  // 1 / 13!
    s = fma(s, r2, -1.0 / 39916800.0);                   // -1 / 11!
    s = fma(s, r2, 1.0 / 362880.0);                      // 1 / 9!
    s = fma(s, r2, -1.0 / 5040.0);
    s = fma(s, r2, 1.0 / 120.0);
    s = fma(s, r2, -1.0 / 6.0);
    s = fma(s * r2, r, r);                               // r + r^3 (...)
    double c = 1.0 / 20922789888000.0;                   // 1 / 16!
    c = fma(c, r2, -1.0 / 87178291200.0);                // -1 / 14!
    c = fma(c, r2, 1.0 / 479001600.0);                   // 1 / 12!
    c = fma(c, r2, -1.0 / 3628800.0);                    // -1 / 10!
    c = fma(c, r2, 1.0 / 40320.0);
    c = fma(c, r2, -1.0 / 720.0);
    c = fma(c, r2, 1.0 / 24.0);
    c = fma(c, r2, -0.5);
    c = fma(c, r2, 1.0);
    const int q = (int)(long long)k & 3;
    const double ss = (q & 1) ? c : s, cc = (q & 1) ? s : c;
    sn = (float)((q & 2) ? -ss : ss);
    cs = (float)(((q + 1) & 2) ? -cc : cc);
}

__global__ void __launch_bounds__(PRE_WARPS * 32, 6) preop_kernel(const __grid_constant__ PreopParams p) {
    __shared__ float cs_s[PRE_ROWS][64];                 // per token: cos[32], sin[32]
    // squares of the key rows, [key warps of the block][PRE_ROWS][260] (row stride 260: lanes on
    // distinct banks); sized by the launch for the key heads a block can hold
    extern __shared__ __align__(16) float sq_dyn[];
    __shared__ float ss_s[PRE_WARPS * PRE_ROWS];         // the key rows' sums of squares, [key slot of the block][token]
    static_assert(PRE_WARPS * PRE_ROWS <= 32, "one warp walks all key rows of a block");
    // Dependent launch: this kernel reads the projections and writes the cache, so it waits for
    // everything in front of it first; the attention kernel behind it may then start at once (it
    // waits itself before it touches the rows appended here).
    pdl_wait();
    pdl_launch_next();
    const PreopSeq &s = p.seq[blockIdx.z];
    const int qh = p.q_heads, kvh = p.kv_heads;
    const int qs = p.skip_q ? 0 : qh;                    // query slots this launch handles
    const int nblk = (qs + 2 * kvh + PRE_WARPS - 1) / PRE_WARPS;
    const int r0 = (blockIdx.x / nblk) * PRE_ROWS;
    if (r0 >= s.rows) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot0 = (blockIdx.x % nblk) * PRE_WARPS, slot = slot0 + warp;
    const int n = min(PRE_ROWS, s.rows - r0);
    const bool active = slot < qs + 2 * kvh;             // (idle warps still help with the angles below)
    const bool is_q = slot < qs, is_k = !is_q && slot < qs + kvh;
    const int h = !active ? 0 : is_q ? slot : is_k ? slot - qs : slot - qs - kvh;
    const void *src = is_q ? s.qg : is_k ? s.k : s.v;
    const size_t pitch = is_q ? (size_t)qh * 512 : (size_t)kvh * 256, off = is_q ? (size_t)h * 512 : (size_t)h * 256;
    __nv_bfloat16 *dst = is_q ? s.q_out : is_k ? s.kc.base : s.vc.base;
    const uint16_t *wn = is_q ? p.q_norm_w : p.k_norm_w;

    // all rows of the warp in flight before the first is touched, and before the angles
    uint4 raw[PRE_ROWS][2];
    int64_t dst_row[PRE_ROWS];
#pragma unroll
    for (int u = 0; u < PRE_ROWS; u++) {
        if (!active) { dst_row[u] = -1; continue; }
        const int r = min(r0 + u, s.rows - 1);
        const size_t first = (size_t)r * pitch + off + lane * 8;
        raw[u][1] = make_uint4(0, 0, 0, 0);
        if (p.io_dtype == DT_BF16) {
            raw[u][0] = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(src) + first));
        } else {
            const uint4 *g = reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(src) + first);
            raw[u][0] = __ldg(g);
            raw[u][1] = __ldg(g + 1);
        }
        dst_row[u] = is_q ? (int64_t)r * qh + h : kv_row(is_k ? s.kc : s.vc, h, s.base_pos + r);
    }
    uint4 w4 = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);     // the norm weights ride along with the rows
    if (active && wn && (is_q || is_k)) w4 = __ldg(reinterpret_cast<const uint4 *>(wn) + lane);
    if (slot0 < qs + kvh) {                              // the block holds a query or key head
        if (warp < n) {
            const int r = r0 + warp;
            // the token's position on all three axes and the dim's axis are fetched side by side
            // (a position looked up through the axis would be a second trip to memory)
            const int32_t p0 = s.pos[r], p1 = s.pos[(size_t)s.rows + r], p2 = s.pos[(size_t)2 * s.rows + r];
            const int ax = p.axis[lane];
            const float ang = __fmul_rn((float)(ax == 0 ? p0 : ax == 1 ? p1 : p2), p.inv_freq[lane]);
            // cosf / sinf of the fp32 angle (qwasar_cpu.c:312-315), correctly rounded: the double
            // functions are exact far beyond float precision, so one rounding gives the float result
            float sn, cs;
            sincos_rounded(ang, sn, cs);
            cs_s[warp][lane] = cs; cs_s[warp][32 + lane] = sn;
            if (s.cs_out && slot0 <= qs && qs < slot0 + PRE_WARPS) {          // the block with key head 0 publishes the table
                s.cs_out[(size_t)r * 64 + lane] = cs; s.cs_out[(size_t)r * 64 + 32 + lane] = sn;
            }
        }
        __syncthreads();
    }
    auto unpack = [&](int u, float (&x)[8]) {
        if (p.io_dtype == DT_BF16) {
            const uint32_t xw[4] = {raw[u][0].x, raw[u][0].y, raw[u][0].z, raw[u][0].w};
#pragma unroll
            for (int i = 0; i < 4; i++) { x[2 * i] = __uint_as_float(xw[i] << 16); x[2 * i + 1] = __uint_as_float(xw[i] & 0xffff0000u); }
        } else {
            x[0] = __uint_as_float(raw[u][0].x); x[1] = __uint_as_float(raw[u][0].y); x[2] = __uint_as_float(raw[u][0].z); x[3] = __uint_as_float(raw[u][0].w);
            x[4] = __uint_as_float(raw[u][1].x); x[5] = __uint_as_float(raw[u][1].y); x[6] = __uint_as_float(raw[u][1].z); x[7] = __uint_as_float(raw[u][1].w);
        }
    };
    // Key rows: the squares are added left to right over the 256 dims like the CPU loop
    // (qwasar_cpu.c:70-72).  The rows' squares go through shared memory and ONE warp walks them, a lane
    // per row -- all key rows of the block side by side (up to PRE_WARPS heads x PRE_ROWS tokens) -- so
    // the 256 dependent additions are issued once per block, not once per key warp: with each key warp
    // walking its own four rows the pre-op of a 4096-token prefill spent 8 of its 10 million
    // instructions here.
    float ss_k[PRE_ROWS];
#pragma unroll
    for (int u = 0; u < PRE_ROWS; u++) ss_k[u] = 0.0f;
    const int k_first = max(slot0, qs), k_last = min(slot0 + PRE_WARPS, qs + kvh);   // key slots of this block: [k_first, k_last)
    if (k_first < k_last) {                              // (the same for the whole block)
        float *sq_mine = sq_dyn + (size_t)(is_k ? slot - k_first : 0) * PRE_ROWS * 260;
        if (is_k) {
#pragma unroll
            for (int u = 0; u < PRE_ROWS; u++) {
                if (u >= n || dst_row[u] < 0) continue;      // warp-uniform
                float x[8];
                unpack(u, x);
                float4 *sq = reinterpret_cast<float4 *>(sq_mine + u * 260 + lane * 8);
                sq[0] = make_float4(__fmul_rn(x[0], x[0]), __fmul_rn(x[1], x[1]), __fmul_rn(x[2], x[2]), __fmul_rn(x[3], x[3]));
                sq[1] = make_float4(__fmul_rn(x[4], x[4]), __fmul_rn(x[5], x[5]), __fmul_rn(x[6], x[6]), __fmul_rn(x[7], x[7]));
            }
        }
        __syncthreads();
        if (warp == 0 && lane < (k_last - k_first) * PRE_ROWS && (lane % PRE_ROWS) < n) {
            const float4 *sq = reinterpret_cast<const float4 *>(sq_dyn + (size_t)lane * 260);   // row (slot lane / PRE_ROWS, token lane % PRE_ROWS)
            float acc = 0.0f;
#pragma unroll 4
            for (int i = 0; i < 64; i++) {
                const float4 v = sq[i];
                acc = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(acc, v.x), v.y), v.z), v.w);
            }
            // ... and turns it into the row's norm factor here, once per row instead of once per lane of its warp
            ss_s[lane] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(acc, 256.0f), p.eps)));
        }
        __syncthreads();
        if (is_k) {
#pragma unroll
            for (int u = 0; u < PRE_ROWS; u++) ss_k[u] = ss_s[(slot - k_first) * PRE_ROWS + u];
        }
    }
    if (!active) return;
    float w[8];
    if (wn && (is_q || is_k)) {
        const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int i = 0; i < 4; i++) { w[2 * i] = __uint_as_float(ww[i] << 16); w[2 * i + 1] = __uint_as_float(ww[i] & 0xffff0000u); }
    }
#pragma unroll
    for (int u = 0; u < PRE_ROWS; u++) {
        if (u >= n || dst_row[u] < 0) continue;          // warp-uniform
        uint4 *out = reinterpret_cast<uint4 *>(dst + dst_row[u] * 256) + lane;
        if (!is_q && !is_k && p.io_dtype == DT_BF16) { *out = raw[u][0]; continue; }      // V, already bf16: a copy
        float x[8];
        unpack(u, x);
        if (is_q || is_k) {
            // RMS norm (qwasar_cpu.c:68-82), then the weight
            float inv;
            if (is_k) {
                inv = ss_k[u];                           // (already the factor, see above)
            } else {
                float ss = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) ss = __fadd_rn(ss, __fmul_rn(x[i], x[i]));
                ss = warp_sum(ss);
                inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 256.0f), p.eps)));
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                x[i] = __fmul_rn(x[i], inv);
                if (wn) x[i] = __fmul_rn(x[i], w[i]);
            }
            // partial RoPE (qwasar_cpu.c:304-319): dims d < 32 in lanes 0-3, their partners d + 32 in lanes 4-7
            // (no branch: every lane does the arithmetic, lanes 8-31 on a dummy angle, and keeps its own value)
            const float *cr = cs_s[u] + 8 * (lane & 3);
            const bool rot = lane < 8, lo = lane < 4;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float other = __shfl_xor_sync(0xffffffffu, x[i], 4);
                const float c = cr[i], sn = lo ? -cr[32 + i] : cr[32 + i];
                // lo' = lo c - hi s, hi' = hi c + lo s (the negation is exact, so the first is the same sum)
                const float y = __fadd_rn(__fmul_rn(x[i], c), __fmul_rn(other, sn));
                x[i] = rot ? y : x[i];
            }
        }
        *out = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
    }
}

}  // namespace

void launch_kv_pack(cudaStream_t s, KvLayer kc, KvLayer vc, void *packed, int kv_heads, int n_tokens, bool unpack) {
    const int64_t rows = (int64_t)kv_heads * 2 * n_tokens;
    if (rows <= 0) return;
    kv_pack_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(kc, vc, reinterpret_cast<uint4 *>(packed), kv_heads, n_tokens, unpack);
    g_launches++;
}
// The small ops start under the kernel in front of them on the stream (each waits for it before it touches memory):
// in the graph's own sequence of eight ops per layer the gaps between launches outweigh the kernels.
template <typename... Params, typename... Args>
static void launch_small(void (*kernel)(Params...), unsigned grid, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(256); cfg.stream = s; cfg.attrs = attr; cfg.numAttrs = g_tune_pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kernel, Params(args)...) == cudaSuccess) g_launches++;
}
void launch_split_heads2(cudaStream_t s, float *a, float *b, const float *src, int rows, int heads, int dim) {
    const int64_t n = (int64_t)rows * heads * dim;
    if (n <= 0) return;
    launch_small(split_heads2_kernel, (unsigned)((n + 255) / 256), s, a, b, src, (int64_t)rows * heads, dim);
}
void launch_rms_norm(cudaStream_t s, float *y, const float *x, const uint16_t *w, int dim, int rows, float eps,
                     float out_scale) {
    if (rows <= 0) return;
    launch_small(rms_norm_kernel, (unsigned)((rows + 7) / 8), s, y, x, w, dim, rows, eps, out_scale);
}
void launch_rope_partial(cudaStream_t s, float *x, const int32_t *pos, const uint8_t *axis, const float *inv_freq,
                         int rows, int heads, int head_dim, int rotary_dim) {
    const int64_t n = (int64_t)rows * heads * (rotary_dim / 2);
    if (n <= 0) return;
    launch_small(rope_partial_kernel, (unsigned)((n + 255) / 256), s, x, pos, axis, inv_freq, rows, heads, head_dim, rotary_dim / 2);
}
void launch_kv_write(cudaStream_t s, KvLayer kc, KvLayer vc, const float *k, const float *v, int rows, int kv_heads,
                     int base_pos) {
    const int n = rows * kv_heads;
    if (n <= 0) return;
    launch_small(kv_write_kernel, (unsigned)((n + 7) / 8), s, kc, vc, k, v, rows, kv_heads, base_pos);
}
void launch_mul_sigmoid(cudaStream_t s, float *y, const float *gate, int64_t n) {
    if (n <= 0) return;
    launch_small(mul_sigmoid_kernel, (unsigned)((n + 255) / 256), s, y, gate, n);
}
void launch_slice_rows(cudaStream_t s, float *dst, const float *src, int rows, int src_stride, int offset, int len) {
    const int64_t n = (int64_t)rows * len;
    if (n <= 0) return;
    launch_small(slice_rows_kernel, (unsigned)((n + 255) / 256), s, dst, src, n, src_stride, offset, len);
}
void launch_f32_to_bf16(cudaStream_t s, __nv_bfloat16 *dst, const float *src, int64_t n) {
    if (n <= 0) return;
    launch_small(f32_to_bf16_kernel, (unsigned)((n + 1023) / 1024), s, dst, src, n);
}
void launch_preop(cudaStream_t s, const PreopParams &p, int max_rows) {
    const int slots = (p.skip_q ? 0 : p.q_heads) + 2 * p.kv_heads;
    if (slots == 0) return;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = cudaLaunchConfig_t();
    cfg.gridDim = dim3((unsigned)((max_rows + PRE_ROWS - 1) / PRE_ROWS) * ((slots + PRE_WARPS - 1) / PRE_WARPS), 1, p.n_seq);
    cfg.blockDim = dim3(PRE_WARPS * 32);
    cfg.dynamicSmemBytes = (size_t)(p.kv_heads < PRE_WARPS ? p.kv_heads : PRE_WARPS) * PRE_ROWS * 260 * sizeof(float);
    cfg.stream = s;
    cfg.attrs = &attr; cfg.numAttrs = g_tune_pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, preop_kernel, p);
    g_launches++;
}

}  // namespace qw
