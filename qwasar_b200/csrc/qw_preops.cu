// Pre- and post-ops of the gated attention node: head split, per-head RMS norm,
// partial RoPE, KV append, sigmoid gate -- as separate kernels behind the
// reference's op signatures, and as one fused kernel for the node.
//
// All of it is HBM-bound element work: one warp owns one 256-wide head row, loads
// and stores are 128 B per warp instruction, and nothing is read twice.
//
// Arithmetic follows the reference's scalar twins operation for operation
// (qwasar_cpu.c:68-82, 304-319, 344-355) with contraction switched off through
// the _rn intrinsics, so results differ from the CPU code only by the order of
// the 256-term sum of squares and by the last bit of cosf/sinf.
#include "qw_kernels.h"

namespace qw {

namespace {

__device__ __forceinline__ float load_io(const void *p, size_t i, int dtype) {
    return dtype == DT_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i])
                            : reinterpret_cast<const float *>(p)[i];
}

// Lane l of a warp holds dims l, l+32, ..., l+224 of a head row, so that the RoPE
// pair (j, j + 32) for j < 32 sits in one lane (x[0], x[1]).
__device__ __forceinline__ void norm8(float (&x)[8], const uint16_t *w, int lane, float eps, float out_scale) {
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) ss = __fadd_rn(ss, __fmul_rn(x[i], x[i]));
    ss = warp_sum(ss);
    const float inv = __fmul_rn(__fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 256.0f), eps))), out_scale);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float t = __fmul_rn(x[i], inv);
        if (w) t = __fmul_rn(t, bf16_bits_to_f32(w[lane + 32 * i]));
        x[i] = t;
    }
}

// Rotates (x[0], x[1]) = dims (lane, lane + 32); rotary_dim == 64 here.
__device__ __forceinline__ void rope64(float (&x)[8], const int32_t *pos, const uint8_t *axis,
                                       const float *inv_freq, int rows, int r, int lane) {
    const float ang = __fmul_rn((float)pos[(size_t)axis[lane] * rows + r], inv_freq[lane]);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    const float lo = x[0], hi = x[1];
    x[0] = __fsub_rn(__fmul_rn(lo, cs), __fmul_rn(hi, sn));
    x[1] = __fadd_rn(__fmul_rn(hi, cs), __fmul_rn(lo, sn));
}

// ---- unfused ops, reference signatures ------------------------------------------------

__global__ void split_heads2_kernel(float *__restrict__ a, float *__restrict__ b, const float *__restrict__ src,
                                    int64_t n_rh, int dim) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // over n_rh * dim
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
    if (i < n) y[i] = __fmul_rn(y[i], __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g[i]))));
}

__global__ void f32_to_bf16_kernel(__nv_bfloat16 *__restrict__ dst, const float *__restrict__ src, int64_t n) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
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

// A 256-wide head row between global memory and the lane layout above (lane l holds dims
// l + 32 i), through a per-warp row buffer in shared memory: global accesses are 16 bytes per
// lane (one or two instructions per row instead of eight 2- or 4-byte ones), and the strided
// shared-memory accesses are conflict-free.
__device__ __forceinline__ void load_row(float (&x)[8], const void *src, size_t first, int dtype, bool vec, uint32_t *buf, int lane) {
    if (!vec) {
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = load_io(src, first + lane + 32 * i, dtype);
    } else if (dtype == DT_BF16) {
        reinterpret_cast<uint4 *>(buf)[lane] = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(src) + first) + lane);
        __syncwarp();
        const uint16_t *h = reinterpret_cast<const uint16_t *>(buf);
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = bf16_bits_to_f32(h[lane + 32 * i]);
    } else {
        const uint4 *g = reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(src) + first);
        reinterpret_cast<uint4 *>(buf)[lane] = __ldg(g + lane);
        reinterpret_cast<uint4 *>(buf)[lane + 32] = __ldg(g + lane + 32);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = __uint_as_float(buf[lane + 32 * i]);
    }
    __syncwarp();
}
__device__ __forceinline__ void store_row_bf16(__nv_bfloat16 *dst, const float (&x)[8], uint32_t *buf, int lane) {
    __nv_bfloat16 *h = reinterpret_cast<__nv_bfloat16 *>(buf);
#pragma unroll
    for (int i = 0; i < 8; i++) h[lane + 32 * i] = __float2bfloat16_rn(x[i]);
    __syncwarp();
    reinterpret_cast<uint4 *>(dst)[lane] = reinterpret_cast<const uint4 *>(buf)[lane];
    __syncwarp();
}

// ---- the fused pre-op ---------------------------------------------------------------------
// grid = (max_rows * ceil(slots / 8), 1, n_seq) with slots = q_heads + 2 * kv_heads; one warp per
// (sequence, row, slot): slot < q_heads is a query head, then the key heads, then the value heads.
__global__ void __launch_bounds__(256) preop_kernel(const __grid_constant__ PreopParams p) {
    __shared__ __align__(16) uint32_t rowbuf[8][256];
    uint32_t *buf = rowbuf[threadIdx.x >> 5];
    const PreopSeq &s = p.seq[blockIdx.z];
    const int nblk = (p.q_heads + 2 * p.kv_heads + 7) / 8;
    const int r = blockIdx.x / nblk;
    if (r >= s.rows) return;
    const int slot = (blockIdx.x % nblk) * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int qh = p.q_heads, kvh = p.kv_heads;
    if (slot >= qh + 2 * kvh) return;

    float x[8];
    if (slot < qh) {
        load_row(x, s.qg, ((size_t)r * qh + slot) * 512, p.io_dtype, p.vec_io != 0, buf, lane);
        norm8(x, p.q_norm_w, lane, p.eps, 1.0f);
        rope64(x, s.pos, p.axis, p.inv_freq, s.rows, r, lane);
        store_row_bf16(s.q_out + ((size_t)r * qh + slot) * 256, x, buf, lane);
    } else if (slot < qh + kvh) {
        const int h = slot - qh;
        load_row(x, s.k, ((size_t)r * kvh + h) * 256, p.io_dtype, p.vec_io != 0, buf, lane);
        norm8(x, p.k_norm_w, lane, p.eps, 1.0f);
        rope64(x, s.pos, p.axis, p.inv_freq, s.rows, r, lane);
        const int64_t row = kv_row(s.kc, h, s.base_pos + r);
        if (row < 0) return;
        store_row_bf16(s.kc.base + row * 256, x, buf, lane);
    } else {
        const int h = slot - qh - kvh;
        const int64_t row = kv_row(s.vc, h, s.base_pos + r);
        if (row < 0) return;
        load_row(x, s.v, ((size_t)r * kvh + h) * 256, p.io_dtype, p.vec_io != 0, buf, lane);
        store_row_bf16(s.vc.base + row * 256, x, buf, lane);
    }
}

}  // namespace

void launch_split_heads2(cudaStream_t s, float *a, float *b, const float *src, int rows, int heads, int dim) {
    const int64_t n = (int64_t)rows * heads * dim;
    if (n <= 0) return;
    split_heads2_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, b, src, (int64_t)rows * heads, dim);
    g_launches++;
}
void launch_rms_norm(cudaStream_t s, float *y, const float *x, const uint16_t *w, int dim, int rows, float eps,
                     float out_scale) {
    if (rows <= 0) return;
    rms_norm_kernel<<<(rows + 7) / 8, 256, 0, s>>>(y, x, w, dim, rows, eps, out_scale);
    g_launches++;
}
void launch_rope_partial(cudaStream_t s, float *x, const int32_t *pos, const uint8_t *axis, const float *inv_freq,
                         int rows, int heads, int head_dim, int rotary_dim) {
    const int64_t n = (int64_t)rows * heads * (rotary_dim / 2);
    if (n <= 0) return;
    rope_partial_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, pos, axis, inv_freq, rows, heads, head_dim,
                                                                     rotary_dim / 2);
    g_launches++;
}
void launch_kv_write(cudaStream_t s, KvLayer kc, KvLayer vc, const float *k, const float *v, int rows, int kv_heads,
                     int base_pos) {
    const int n = rows * kv_heads;
    if (n <= 0) return;
    kv_write_kernel<<<(n + 7) / 8, 256, 0, s>>>(kc, vc, k, v, rows, kv_heads, base_pos);
    g_launches++;
}
void launch_mul_sigmoid(cudaStream_t s, float *y, const float *gate, int64_t n) {
    if (n <= 0) return;
    mul_sigmoid_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(y, gate, n);
    g_launches++;
}
void launch_f32_to_bf16(cudaStream_t s, __nv_bfloat16 *dst, const float *src, int64_t n) {
    if (n <= 0) return;
    f32_to_bf16_kernel<<<(unsigned)((n + 1023) / 1024), 256, 0, s>>>(dst, src, n);
    g_launches++;
}
void launch_preop(cudaStream_t s, const PreopParams &p, int max_rows) {
    const int slots = p.q_heads + 2 * p.kv_heads;
    dim3 grid((unsigned)max_rows * ((slots + 7) / 8), 1, p.n_seq);
    preop_kernel<<<grid, 256, 0, s>>>(p);
    g_launches++;
}

}  // namespace qw
