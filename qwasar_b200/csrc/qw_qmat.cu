// The 4-bit affine product on either side of the attention node (q/k/v projections before it,
// o_proj after it): y[r][o] = sum_i (scale * nibble + bias) * x[r][i], MLX layout -- w U32
// [n, k/8] (element i of row o in word i/8 at bit 4 (i % 8)), bf16 scales and biases per group of
// 32 or 64 elements (qwasar_gpu.h:84-103; CPU twin qw_cpu_qmv_q4, qwasar_cpu.c:36-63).
//
// One kernel for every row count: a block of 8 warps takes 8 output rows of w (one per warp) and a
// tile of up to QM_ROWS tokens, so a weight word is fetched and unpacked once per tile; a lane
// unpacks one word (8 elements) per step and reads the matching 32 bytes of every token's x, all
// of it coalesced.  fp32 throughout; the k terms of an output are added lane by lane and then
// across the warp (the reference's test bounds that reordering at 2e-6 of the sum of absolute
// terms, tests/test_qmv.c:31-50,129).  A first correct version: weight-bandwidth-bound at one
// token, not on tensor cores for many.
#include <algorithm>
#include "qw_kernels.h"

namespace qw {

namespace {

constexpr int QM_ROWS = 8;

__global__ void __launch_bounds__(256) qmat_q4_kernel(float *__restrict__ y, const float *__restrict__ x, const uint32_t *__restrict__ w,
                                                      const uint16_t *__restrict__ scales, const uint16_t *__restrict__ biases, int k,
                                                      int n, int rows, int group) {
    const int o = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int r0 = blockIdx.y * QM_ROWS, nr = min(QM_ROWS, rows - r0);
    if (o >= n) return;
    const int words = k >> 3, groups = k / group, wpg = group >> 3;           // words per group: 4 or 8
    const uint32_t *wr = w + (size_t)o * words;
    const uint16_t *sr = scales + (size_t)o * groups, *br = biases + (size_t)o * groups;
    float acc[QM_ROWS];
#pragma unroll
    for (int r = 0; r < QM_ROWS; r++) acc[r] = 0.0f;
    for (int wi = lane; wi < words; wi += 32) {
        const uint32_t word = wr[wi];
        const float sc = bf16_bits_to_f32(sr[wi / wpg]), bi = bf16_bits_to_f32(br[wi / wpg]);
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = __fadd_rn(__fmul_rn(sc, (float)((word >> (4 * e)) & 0xFu)), bi);
#pragma unroll
        for (int r = 0; r < QM_ROWS; r++) {
            if (r < nr) {
                const float4 *xp = reinterpret_cast<const float4 *>(x + (size_t)(r0 + r) * k + (size_t)wi * 8);
                const float4 a = xp[0], b = xp[1];
                float s = acc[r];
                s = __fadd_rn(s, __fmul_rn(v[0], a.x)); s = __fadd_rn(s, __fmul_rn(v[1], a.y));
                s = __fadd_rn(s, __fmul_rn(v[2], a.z)); s = __fadd_rn(s, __fmul_rn(v[3], a.w));
                s = __fadd_rn(s, __fmul_rn(v[4], b.x)); s = __fadd_rn(s, __fmul_rn(v[5], b.y));
                s = __fadd_rn(s, __fmul_rn(v[6], b.z)); s = __fadd_rn(s, __fmul_rn(v[7], b.w));
                acc[r] = s;
            }
        }
    }
#pragma unroll
    for (int r = 0; r < QM_ROWS; r++) {
        const float s = warp_sum(acc[r]);
        if (lane == 0 && r < nr) y[(size_t)(r0 + r) * n + o] = s;
    }
}

// One or two tokens: the product is a stream of weight bytes, so the kernel is built around the
// loads.  A lane fetches 16 bytes of a weight row (4 words = 32 elements, inside one scale group)
// per step, four steps of a 4096-element chunk of k in flight at once; the tokens' chunk of x sits
// in shared memory, 32 floats per 36-float slot so that the lanes' 16-byte reads of their slots
// fall on different banks; a warp takes QV_OUTS output rows one after the other over the same
// staged chunk.  What the SMs pay for here is the unpacking, so scale and bias stay outside the
// sum over a slot (a slot lies inside one scale group).
constexpr int QV_ROWS = 2, QV_OUTS = 4, QV_KC = 4096, QV_SLOTS = QV_KC / 32, QV_PAD = 36;
__device__ __forceinline__ void qmv_q4_block(float *__restrict__ y, const float *__restrict__ x, const uint32_t *__restrict__ w,
                                             const uint16_t *__restrict__ scales, const uint16_t *__restrict__ biases, int k,
                                             int n, int rows, int group, int block, int row_block) {
    __shared__ __align__(16) float xs[QV_ROWS][QV_SLOTS][QV_PAD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int o0 = (block * 8 + warp) * QV_OUTS;
    const int r0 = row_block * QV_ROWS, nr = min(QV_ROWS, rows - r0);
    const int words = k >> 3, groups = k / group;
    float acc[QV_OUTS][QV_ROWS];
#pragma unroll
    for (int j = 0; j < QV_OUTS; j++)
#pragma unroll
        for (int r = 0; r < QV_ROWS; r++) acc[j][r] = 0.0f;
    for (int kc0 = 0; kc0 < k; kc0 += QV_KC) {
        const int kc = min(QV_KC, k - kc0), slots = kc >> 5, q4 = kc >> 2;      // k is a multiple of 32
        __syncthreads();                                                        // the chunk before has been consumed
        for (int idx = threadIdx.x; idx < nr * q4; idx += 256) {
            const int r = idx / q4, e = (idx - r * q4) * 4;
            *reinterpret_cast<float4 *>(&xs[r][e >> 5][e & 31]) = *reinterpret_cast<const float4 *>(x + (size_t)(r0 + r) * k + kc0 + e);
        }
        __syncthreads();
        // the sum of every slot's 32 inputs, kept in the slot's padding: scale and bias then come
        // out of the inner sum, sum_e (sc * nib_e + bi) * x_e = sc * sum_e nib_e * x_e + bi * sum_e x_e
        for (int idx = threadIdx.x; idx < nr * slots; idx += 256) {
            const int r = idx / slots, q = idx - r * slots;
            float sum = 0.0f;
#pragma unroll
            for (int e = 0; e < 32; e++) sum += xs[r][q][e];
            xs[r][q][32] = sum;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < QV_OUTS; j++) {
            const int o = o0 + j;
            if (o >= n) continue;                                               // warp-uniform
            const uint4 *wr = reinterpret_cast<const uint4 *>(w + (size_t)o * words + (kc0 >> 3));
            const uint16_t *sr = scales + (size_t)o * groups, *br = biases + (size_t)o * groups;
            uint4 wv[4];
            float sc[4], bi[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int q = lane + 32 * i;
                wv[i] = make_uint4(0, 0, 0, 0); sc[i] = 0.0f; bi[i] = 0.0f;
                if (q < slots) {
                    wv[i] = __ldg(wr + q);
                    const int gi = (kc0 + q * 32) / group;
                    sc[i] = bf16_bits_to_f32(sr[gi]); bi[i] = bf16_bits_to_f32(br[gi]);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int q = lane + 32 * i;
                if (q >= slots) continue;
                const uint32_t ww[4] = {wv[i].x, wv[i].y, wv[i].z, wv[i].w};
#pragma unroll
                for (int r = 0; r < QV_ROWS; r++) {
                    if (r >= nr) continue;
                    float s1 = 0.0f;
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const float4 a = *reinterpret_cast<const float4 *>(&xs[r][q][u * 8]);
                        const float4 b = *reinterpret_cast<const float4 *>(&xs[r][q][u * 8 + 4]);
                        const uint32_t word = ww[u];
                        s1 = fmaf((float)(word & 0xFu), a.x, s1);
                        s1 = fmaf((float)((word >> 4) & 0xFu), a.y, s1);
                        s1 = fmaf((float)((word >> 8) & 0xFu), a.z, s1);
                        s1 = fmaf((float)((word >> 12) & 0xFu), a.w, s1);
                        s1 = fmaf((float)((word >> 16) & 0xFu), b.x, s1);
                        s1 = fmaf((float)((word >> 20) & 0xFu), b.y, s1);
                        s1 = fmaf((float)((word >> 24) & 0xFu), b.z, s1);
                        s1 = fmaf((float)(word >> 28), b.w, s1);
                    }
                    float t = acc[j][r];
                    t = fmaf(sc[i], s1, t);
                    t = fmaf(bi[i], xs[r][q][32], t);
                    acc[j][r] = t;
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < QV_OUTS; j++)
#pragma unroll
        for (int r = 0; r < QV_ROWS; r++) {
            const float t = warp_sum(acc[j][r]);
            if (lane == 0 && r < nr && o0 + j < n) y[(size_t)(r0 + r) * n + o0 + j] = t;
        }
}

__global__ void __launch_bounds__(256) qmv_q4_kernel(float *__restrict__ y, const float *__restrict__ x, const uint32_t *__restrict__ w,
                                                     const uint16_t *__restrict__ scales, const uint16_t *__restrict__ biases, int k,
                                                     int n, int rows, int group) {
    qmv_q4_block(y, x, w, scales, biases, k, n, rows, group, blockIdx.x, blockIdx.y);
}

// Up to four one-token products that share their input (the q, k, v and indexer projections of one
// token, qwasar_gpu.h:105-109) as ONE launch: the blocks of all parts laid end to end.
__global__ void __launch_bounds__(256) qmv_q4_multi_kernel(const __grid_constant__ QmvMulti m) {
    int part = 0, block = blockIdx.x;
    while (part + 1 < m.count && block >= m.blocks[part]) { block -= m.blocks[part]; part++; }
    qmv_q4_block(m.y[part], m.x, m.w[part], m.scales[part], m.biases[part], m.k, m.n[part], 1, m.group, block, 0);
}

// One to four tokens, the weights streamed once, the arithmetic on the INTEGER tensor path.
//
// Why integers: at one token the product is bound by instruction issue, not by memory -- turning a
// nibble into a float costs the conversion unit a quarter-rate instruction (or a permute on the
// half-rate logic pipe) and every weight one multiply-add: 5 to 7 instructions per weight, 0.17 to
// 0.21 of the memory bandwidth however x is staged (shared memory, or registers with prefetch).
// mma.sync.m16n8k32.u8.s8 takes the nibbles as they are -- `w & 0x0F0F0F0F` IS an A fragment
// register, 3 instructions per 8 weights -- and adds in int32 without rounding.  x becomes integers
// exactly: each token is scaled by a power of two so that max |x| lands in [2^28, 2^29), rounded to
// an int32 q (every element within 2^-6 of the maximum keeps its full mantissa), and q is cut into
// four balanced base-256 digits, one column of B each: a token owns four of the eight columns, so
// one instruction carries two tokens and a launch two or (two instructions per step over the same
// A fragments) four.  Per group of 64 weights the digit sums come out of the
// accumulators exactly, are combined pairwise in int32, and meet the group's scale in one fp32
// multiply-add per row; the bias meets the group's sum of q.  What is left of rounding is the fp32
// sum over groups and warps, far inside the reference's bound (2e-6 of the sum of absolute terms,
// tests/test_qmv.c:31-50,129).
//
// Layout of the work: a tile is 16 output rows by all of k.  One producer warp brings a tile's
// rows (and their scales and biases) into shared memory with ten bulk copies -- long bursts for
// DRAM, and no register or issue slot of the consumers is spent on loads; up to four tiles are in
// flight per block.  The consumer warps split k, 8 groups each: a quad of lanes takes one group of
// one row, so that an instruction's 32 k-positions lie in one group; a warp's fragments of x stay
// in its registers for the whole launch, its 8 scales of a row are one 16-byte read.  A last warp
// adds the consumers' partial sums of a tile up and writes y, behind a barrier of its own, so no
// consumer ever waits for another.  Blocks are persistent, one per SM, tiles strided over them; x is
// quantised while the first tiles travel (it is asked for before the second tile is, or it would
// queue behind them).  A token with an infinity or a NaN in x yields NaN for all its outputs.
// From three tokens on the digits are cut once, by a small kernel ahead of this one, and every block
// copies them in: cut in each block they cost the four-token product 7.8 of its 16.7 us (13.0 us with
// the kernel ahead, whose blocks are small enough to become resident beside this kernel's and so start
// the moment the kernel before ends; at one and two tokens the second launch costs more than it
// saves, 12.0 against 10.1 us).
//
// What was measured on the way (k 5120, n 12288, one token, 35 MB per launch, back-to-back launches
// over eight weight sets): lanes loading 8 bytes each, one group of one row per quad, 1.0 TB/s (the
// memory system was handed 32-byte sectors of eight rows per request); one bulk copy per row, 48 a
// tile, 2.5 TB/s with the arithmetic switched off (a copy costs the unit a fixed time); a block-wide
// barrier per tile and x in shared memory, 2.3 TB/s; this form 3.3 TB/s, of which the stream itself
// runs at DRAM speed (a tile per SM every 0.95 us) and the rest is the launch gap (2.2 us), the first
// tile's latency (2.4 us) and the last tile's arithmetic (1.2 us).
constexpr int QI_MAXW = 14, QI_MAXW4 = 12, QI_MAXS = 4, QI_ITEMS = 4, QI_PER = 8, QI_SLOTS = 4;   // warps, stages, 8-element items per thread, groups per warp, slots of partial sums
struct QmvJob {
    float *y[4];
    const uint32_t *w[4];
    const uint16_t *scales[4], *biases[4];
    const float *x;
    const unsigned char *xq;                                   // x already cut into digits (qmv_quant_x_kernel), or null
    int *status;
    int32_t n[4], tile_end[4];                                 // running total of 16-row tiles over the parts
    int32_t count, k, tokens, per, tiles, stages, w_stride;   // w_stride: bytes from one staged pair of rows to the next
};

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// global -> shared bulk copy (untiled; both addresses and the size multiples of 16 bytes), completing on `bar`
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// asks for a range to be brought into L2 (no data reaches the SM: safe before the kernel's dependencies are met)
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint2 lds_u2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds_u4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void consumer_sync(int threads) { asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory"); }

// Eight elements of x, scaled, as balanced base-256 digits in B-fragment order, and the two halves of their sum.
// q + 0x00808080 has the balanced base-256 digits of q, each plus 128, as its low three bytes and the top
// digit as its (signed) high byte: the xor takes the 128s off again.  Then two 4 x 4 byte transposes put
// digit p of elements 0, 2, 4, 6 into one B register and of 1, 3, 5, 7 into the other.
__device__ __forceinline__ void cut_digits(const float (&v)[8], float scale, uint2 (&col)[4], int &sum_hi, int &sum_lo) {
    uint32_t z[8];
    sum_hi = 0; sum_lo = 0;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int q = __float2int_rn(v[j] * scale);
        sum_hi += q >> 8; sum_lo += q & 255;
        z[j] = (uint32_t)(q + 0x00808080) ^ 0x00808080u;
    }
    {
        const uint32_t t0 = __byte_perm(z[0], z[2], 0x5140), t1 = __byte_perm(z[0], z[2], 0x7362);
        const uint32_t u0 = __byte_perm(z[4], z[6], 0x5140), u1 = __byte_perm(z[4], z[6], 0x7362);
        col[0].x = __byte_perm(t0, u0, 0x5410); col[1].x = __byte_perm(t0, u0, 0x7632);
        col[2].x = __byte_perm(t1, u1, 0x5410); col[3].x = __byte_perm(t1, u1, 0x7632);
    }
    {
        const uint32_t t0 = __byte_perm(z[1], z[3], 0x5140), t1 = __byte_perm(z[1], z[3], 0x7362);
        const uint32_t u0 = __byte_perm(z[5], z[7], 0x5140), u1 = __byte_perm(z[5], z[7], 0x7362);
        col[0].y = __byte_perm(t0, u0, 0x5410); col[1].y = __byte_perm(t0, u0, 0x7632);
        col[2].y = __byte_perm(t1, u1, 0x5410); col[3].y = __byte_perm(t1, u1, 0x7632);
    }
}

// The digits of x for the kernel below, cut once per product instead of once per block of it: a block per token,
// a thread per 8-element chunk.  Tokens go four to a blob -- [16 columns][k / 8 + 4] chunks in the order the kernel
// below keeps them in shared memory, [4][k / 64] sums of q per group, [4] max |x| bits -- and a blob's missing tokens
// are written as zeros.  (Cutting them in every block cost the four-token product 7.8 of its 16.8 us.)
constexpr int QQ_THREADS = 256, QQ_ITEMS = 4;                 // (few threads and registers: a block fits beside a block of the product before)
__global__ void __launch_bounds__(QQ_THREADS) qmv_quant_x_kernel(const float *__restrict__ x, unsigned char *__restrict__ blobs, int rows, int k, unsigned blob_bytes) {
    __shared__ uint32_t s_m[QQ_THREADS / 32];
    const int t = blockIdx.x, r = t & 3, words = k >> 3, groups = k >> 6, xcol = words + 4;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int carried = min(4, rows - (t & ~3)) > 2 ? 4 : 2;    // columns of tokens the blob's consumer multiplies by
    unsigned char *blob = blobs + (size_t)(t >> 2) * blob_bytes;
    uint2 *xs = reinterpret_cast<uint2 *>(blob);
    float *xg = reinterpret_cast<float *>(blob + 128u * (unsigned)xcol);
    uint32_t *xmax = reinterpret_cast<uint32_t *>(xg + 4 * groups);
    pdl_launch_next();                                          // the product may start fetching its weights
    pdl_wait();                                                 // x may come from the kernel before, which may also still read the blobs
    float v[QQ_ITEMS][8];
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < QQ_ITEMS; i++) {
        const int c = tid + i * QQ_THREADS;
#pragma unroll
        for (int j = 0; j < 8; j++) v[i][j] = 0.0f;
        if (t < rows && c < words) {
            const int e0 = (c >> 3) * 64 + (c & 3) * 16 + ((c >> 2) & 1) * 8;      // chunk c = (group, word of the lane, lane-in-quad)
            const float4 a = __ldg(reinterpret_cast<const float4 *>(x + (size_t)t * k + e0));
            const float4 b = __ldg(reinterpret_cast<const float4 *>(x + (size_t)t * k + e0 + 4));
            v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w; v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
        }
    }
#pragma unroll
    for (int i = 0; i < QQ_ITEMS; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) m = max(m, __float_as_uint(v[i][j]) & 0x7fffffffu);
#pragma unroll
    for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) s_m[warp] = m;
    __syncthreads();
    m = 0;
#pragma unroll
    for (int q = 0; q < QQ_THREADS / 32; q++) m = max(m, s_m[q]);
    const int e = min(max((int)(m >> 23), 29), 254);
    const float scale = __uint_as_float((uint32_t)(282 - e) << 23);   // max |x| * scale in [2^28, 2^29); the adding warp undoes it
#pragma unroll
    for (int i = 0; i < QQ_ITEMS; i++) {
        const int c = tid + i * QQ_THREADS;
        if (i * QQ_THREADS >= words) break;                      // (the same for every thread; words is a multiple of 64)
        uint2 col[4];
        int sum_hi, sum_lo;
        cut_digits(v[i], scale, col, sum_hi, sum_lo);
        // the group's sum of q: its 8 chunks sit in 8 neighbouring lanes
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) { sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, o); sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, o); }
        if (c < words) {
            if (r < carried) {
#pragma unroll
                for (int p = 0; p < 4; p++) xs[(size_t)(r * 4 + p) * xcol + c] = col[p];
            }
            if ((c & 7) == 0) xg[r * groups + (c >> 3)] = fmaf((float)sum_hi, 256.0f, (float)sum_lo);
        }
    }
    if (tid == 0) xmax[r] = m;
}

// NB = 1: up to two tokens (the eight B columns of one instruction per step); NB = 2: up to four (two instructions per
// step over the same A fragments: the weights of a speculative verify's rows are streamed once, not once per pair).
// PRE: the digits of x come ready from qmv_quant_x_kernel (one bulk copy) instead of being cut by every block.
template <int NB, bool PRE>
__global__ void __launch_bounds__(NB == 1 ? (QI_MAXW + 2) * 32 : (QI_MAXW4 + 2) * 32, 1) qmv_imma_q4_kernel(const __grid_constant__ QmvJob job) {
    constexpr int GROUP = 64, NT = 2 * NB;                      // tokens a launch can carry
    extern __shared__ __align__(128) unsigned char qmv_smem[];
    __shared__ uint64_t full[QI_MAXS], empty[QI_MAXS], done[QI_SLOTS], pfree[QI_SLOTS], xbar;
    __shared__ uint32_t s_max[QI_MAXW][4];
    __shared__ int s_abort;
    const int k = job.k, groups = k / GROUP, words = k >> 3, W = (blockDim.x >> 5) - 2, tokens = job.tokens, S = job.stages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3, CT = W * 32;
    float *xg = reinterpret_cast<float *>(qmv_smem);            // [4][groups] sums of q (rows >= tokens: 0), [4] max |x| bits
    const uint32_t *xmax = reinterpret_cast<const uint32_t *>(xg + 4 * groups);
    float *part = xg + 4 * groups + 4;                              // [slot][W][16 rows][NB][4 column pairs]
    float *pbias = part + QI_SLOTS * W * 64 * NB;               // [slot][W][16 rows][4 tokens]
    const uint32_t w_bytes = (uint32_t)(k >> 1), s_bytes = (uint32_t)(groups * 2), stage_bytes = 8u * job.w_stride + 32u * s_bytes;
    unsigned char *stage0 = qmv_smem + (((size_t)groups * 16 + 16 + (size_t)W * 64 * 4 * (NB + 1) * QI_SLOTS + 127) & ~(size_t)127);
    // the quantised x, [8 NB columns][k / 8 chunks of 8 elements, + 4] in fragment order (the + 4 puts the columns 8
    // banks apart: a fragment read then covers all banks, and a chunk's writer stores next to its neighbours'), borrows
    // the LAST NB stages until the consumers hold their fragments in registers (a stage is larger: 9 k bytes against 8 k)
    const int xcol = words + 4;
    uint2 *xs = reinterpret_cast<uint2 *>(stage0 + (size_t)(S - NB) * stage_bytes);
    const int tiles = job.tiles;
    const int my_tiles = (int)blockIdx.x < tiles ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    auto locate = [&](int tile, int &part_i, int &base) {
        part_i = 0; base = 0;
        while (part_i + 1 < job.count && tile >= job.tile_end[part_i]) { base = job.tile_end[part_i]; part_i++; }
    };

    if (tid == 0) {
        s_abort = 0;
        for (int i = 0; i < S; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], W); }
        for (int i = 0; i < QI_SLOTS; i++) { mbar_init(&done[i], W); mbar_init(&pfree[i], 1); }
        mbar_init(&xbar, 1);
        mbar_fence_init();
    }
    if (PRE && warp == W) {
        // while the kernel that cuts x into digits still runs: the first tiles on their way into L2
        for (int it = 0; it < min(my_tiles, S); it++) {
            const int tile = blockIdx.x + it * gridDim.x;
            int pi, base; locate(tile, pi, base);
            const int row0 = (tile - base) * 16, rows_here = min(16, job.n[pi] - row0);
            if (lane < 8 && 2 * lane < rows_here)
                bulk_prefetch_l2(job.w[pi] + (size_t)(row0 + 2 * lane) * words, (uint32_t)min(2, rows_here - 2 * lane) * w_bytes);
            else if (lane == 8) bulk_prefetch_l2(job.scales[pi] + (size_t)row0 * groups, (uint32_t)rows_here * s_bytes);
            else if (lane == 9) bulk_prefetch_l2(job.biases[pi] + (size_t)row0 * groups, (uint32_t)rows_here * s_bytes);
        }
    }
    __syncthreads();
    pdl_wait();                                                 // x may come from the kernel before; nothing is written yet
    pdl_launch_next();

    if (warp == W) {
        // ---- producer: a tile's 16 rows of weights, 16 rows of scales, 16 of biases per stage -------
        // Ten copies per tile: the rows of a tile follow one another in memory, so the weights go pair of
        // rows by pair of rows (the pairs 8 banks apart in shared memory: the 8 rows a fragment load touches
        // then cover all 32 banks in two passes, the least an 8-byte load per lane takes), scales and biases
        // as one block each.  (One copy per row -- 48 a tile -- held the whole kernel to 2.5 TB/s with the
        // arithmetic switched off: a copy costs the unit a fixed time whatever its size.)  Only a part's last
        // tile, when it has fewer than 16 rows, is copied row by row, the missing rows filled with the last.
        if (PRE && lane == 0) {                                  // the digits of x, then the sums and maxima: ahead of the weights
            const uint32_t xs_bytes = 64u * NB * (uint32_t)xcol, aux_bytes = 16u * groups + 16u;
            mbar_expect_tx(&xbar, xs_bytes + aux_bytes);
            bulk_load(xs, job.xq, xs_bytes, &xbar);
            bulk_load(xg, job.xq + 128u * (uint32_t)xcol, aux_bytes, &xbar);
        }
        for (int it = 0; it < my_tiles; it++) {
            const int st = it % S, tile = blockIdx.x + it * gridDim.x;
            if (!PRE && it == 1) asm volatile("bar.sync 2, %0;" ::"r"(CT + 32) : "memory");   // the consumers have asked for x
            if (it == S - NB) asm volatile("bar.sync 3, %0;" ::"r"(CT + 32) : "memory"); // ... and are done with the borrowed stages
            if (it >= S) mbar_wait_hot(&empty[st], ((it / S) - 1) & 1, &s_abort, job.status, QW_ST_SLOT_TIMEOUT);
            int pi, base; locate(tile, pi, base);
            const int row0 = (tile - base) * 16;
            unsigned char *dst = stage0 + (size_t)st * stage_bytes, *dst_s = dst + 8u * job.w_stride;
            if (lane == 0) mbar_expect_tx(&full[st], 16u * w_bytes + 32u * s_bytes);
            __syncwarp();
            if (row0 + 16 <= job.n[pi]) {
                if (lane < 8) bulk_load(dst + (size_t)lane * job.w_stride, job.w[pi] + (size_t)(row0 + 2 * lane) * words, 2u * w_bytes, &full[st]);
                else if (lane == 8) bulk_load(dst_s, job.scales[pi] + (size_t)row0 * groups, 16u * s_bytes, &full[st]);
                else if (lane == 9) bulk_load(dst_s + 16u * s_bytes, job.biases[pi] + (size_t)row0 * groups, 16u * s_bytes, &full[st]);
            } else {
                const int row = min(row0 + (lane & 15), job.n[pi] - 1);
                if (lane < 16) bulk_load(dst + (size_t)(lane >> 1) * job.w_stride + (lane & 1) * w_bytes, job.w[pi] + (size_t)row * words, w_bytes, &full[st]);
                bulk_load(dst_s + (size_t)lane * s_bytes, (lane < 16 ? job.scales[pi] : job.biases[pi]) + (size_t)row * groups, s_bytes, &full[st]);
            }
        }
        if (!PRE && my_tiles < 2) asm volatile("bar.sync 2, %0;" ::"r"(CT + 32) : "memory");
        if (my_tiles <= S - NB) asm volatile("bar.sync 3, %0;" ::"r"(CT + 32) : "memory");
        return;
    }
    if (warp == W + 1) {
        // ---- the warp that adds a tile up: 16 rows x 2 NB tokens, NB per lane, over the W warps' partial sums ----
        const int row = lane >> 1;
        float inv[NB];
        bool bad[NB];
        for (int it = 0; it < my_tiles; it++) {
            const int st = it % QI_SLOTS, tile = blockIdx.x + it * gridDim.x;
            mbar_wait_hot(&done[st], (it / QI_SLOTS) & 1, &s_abort, job.status, QW_ST_MMA_TIMEOUT);
            if (it == 0) {                                       // (the consumers' maxima are complete once a tile is)
                if (PRE) mbar_wait_hot(&xbar, 0, &s_abort, job.status, QW_ST_TMA_TIMEOUT);
#pragma unroll
                for (int u = 0; u < NB; u++) {
                    uint32_t m = 0;
                    if (PRE) m = xmax[(lane & 1) + 2 * u];
                    else for (int q = 0; q < W; q++) m = max(m, s_max[q][(lane & 1) + 2 * u]);
                    const int e = (int)(m >> 23);
                    bad[u] = e == 255;
                    inv[u] = __uint_as_float((uint32_t)(min(max(e, 29), 254) - 28) << 23);
                }
            }
            int pi, base; locate(tile, pi, base);
            const int o = (tile - base) * 16 + row;
#pragma unroll
            for (int u = 0; u < NB; u++) {
                const int t = (lane & 1) + 2 * u;                // token; its digit pairs are columns (t & 1) * 2, + 1 of block u
                const float *a = part + (size_t)st * W * 64 * NB + row * 4 * NB + u * 4 + (t & 1) * 2;
                const float *bq = pbias + (size_t)st * W * 64 + row * 4 + t;
                float lo = 0.0f, hi = 0.0f, bs = 0.0f;
                for (int q = 0; q < W; q++) { lo += a[q * 64 * NB]; hi += a[q * 64 * NB + 1]; bs += bq[q * 64]; }
                if (t < tokens && o < job.n[pi])
                    job.y[pi][(size_t)t * job.n[pi] + o] = bad[u] ? __uint_as_float(0x7fc00000u) : inv[u] * (fmaf(65536.0f, hi, lo) + bs);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&pfree[st]);             // the slot of partial sums may be written again
        }
        return;
    }

    if constexpr (PRE) {
        mbar_wait_hot(&xbar, 0, &s_abort, job.status, QW_ST_TMA_TIMEOUT);
    } else {
    // ---- x -> integers (the consumer warps, while the first tiles travel) -------------------------
    // An item is 8 consecutive elements of one token (a chunk: what one lane feeds one instruction);
    // a thread keeps its items in registers between the pass that finds max |x| and the one that cuts
    // the digits, so x is read once.  (The host side checks that QI_ITEMS items per thread suffice.)
    const int items = words * tokens;
    float xv[QI_ITEMS * NB][8];
    uint32_t mt[NT];
#pragma unroll
    for (int u = 0; u < NT; u++) mt[u] = 0;
#pragma unroll
    for (int i = 0; i < QI_ITEMS * NB; i++) {
        const int it = tid + i * CT;
#pragma unroll
        for (int j = 0; j < 8; j++) xv[i][j] = 0.0f;
        if (it < items) {
            const int t = it / words, c = it - t * words;
            const int e0 = (c >> 3) * GROUP + (c & 3) * 16 + ((c >> 2) & 1) * 8;   // chunk c = (group, word of the lane, lane-in-quad)
            const float4 a = __ldg(reinterpret_cast<const float4 *>(job.x + (size_t)t * k + e0));
            const float4 b = __ldg(reinterpret_cast<const float4 *>(job.x + (size_t)t * k + e0 + 4));
            xv[i][0] = a.x; xv[i][1] = a.y; xv[i][2] = a.z; xv[i][3] = a.w; xv[i][4] = b.x; xv[i][5] = b.y; xv[i][6] = b.z; xv[i][7] = b.w;
        }
    }
    // x is asked for before the weights: behind three stages of weight traffic it would arrive last
    asm volatile("bar.arrive 2, %0;" ::"r"(CT + 32) : "memory");
#pragma unroll
    for (int i = 0; i < QI_ITEMS * NB; i++) {
        const int it = tid + i * CT;
        if (it < items) {
            uint32_t m = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) m = max(m, __float_as_uint(xv[i][j]) & 0x7fffffffu);
            const int t = it / words;
#pragma unroll
            for (int u = 0; u < NT; u++) if (t == u) mt[u] = max(mt[u], m);
        }
    }
#pragma unroll
    for (int u = 0; u < NT; u++) {
#pragma unroll
        for (int o = 16; o; o >>= 1) mt[u] = max(mt[u], __shfl_xor_sync(0xffffffffu, mt[u], o));
        if (lane == 0) s_max[warp][u] = mt[u];
    }
    for (int i = tokens * groups + tid; i < 4 * groups; i += CT) xg[i] = 0.0f;
    consumer_sync(CT);
    float scale[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) {
        uint32_t m = 0;
        for (int q = 0; q < W; q++) m = max(m, s_max[q][t]);
        const int e = min(max((int)(m >> 23), 29), 254);
        scale[t] = __uint_as_float((uint32_t)(282 - e) << 23);  // max |x| * scale in [2^28, 2^29); the adding warp undoes it
    }
#pragma unroll
    for (int i = 0; i < QI_ITEMS * NB; i++) {
        if (i * CT >= items) break;                              // (the same for every thread)
        const int it = tid + i * CT;
        const bool live = it < items;
        const int t = live ? it / words : 0, c = live ? it - t * words : 0;
        float sc_t = scale[0];
#pragma unroll
        for (int u = 1; u < NT; u++) if (t == u) sc_t = scale[u];
        uint2 col[4];
        int sum_hi, sum_lo;
        cut_digits(xv[i], sc_t, col, sum_hi, sum_lo);
        // the group's sum of q: its 8 chunks sit in 8 neighbouring lanes
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) { sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, o); sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, o); }
        if (live) {
#pragma unroll
            for (int p = 0; p < 4; p++) xs[(size_t)(t * 4 + p) * xcol + c] = col[p];
            if (t == 0)                                          // the columns of tokens this launch does not carry: zeros
                for (int p = 4 * tokens; p < 8 * NB; p++) xs[(size_t)p * xcol + c] = make_uint2(0u, 0u);
            if ((c & 7) == 0) xg[t * groups + (c >> 3)] = fmaf((float)sum_hi, 256.0f, (float)sum_lo);
        }
    }
    consumer_sync(CT);
    }

    // ---- the product ---------------------------------------------------------------------------
    // A warp owns 8 consecutive groups of k for every tile: their B fragments (the digits of x) and sums
    // of q stay in registers, its 8 scales and 8 biases of a row are one 16-byte read each, and shared
    // memory is addressed through 32-bit window offsets (with generic pointers the address arithmetic of
    // the reads outweighed the arithmetic they feed).  No block-wide barrier: a warp hands its partial
    // sums to the adding warp through the stage's `done` barrier and goes on to the next tile.
    const int g0 = warp * QI_PER;
    uint2 bx[QI_PER][NB][2];
    float xsum[QI_PER];
#pragma unroll
    for (int i = 0; i < QI_PER; i++) {
#pragma unroll
        for (int u = 0; u < NB; u++) {
            const uint2 *xb = xs + (size_t)(gid + 8 * u) * xcol + (g0 + i) * 8 + tig;   // chunk (group, word 0 / 1 of the lane, lane-in-quad)
            bx[i][u][0] = xb[0]; bx[i][u][1] = xb[4];
        }
        xsum[i] = xg[tig * groups + g0 + i];
    }
    fence_proxy_async();                                           // (our reads of it, before the bulk copies' writes)
    asm volatile("bar.arrive 3, %0;" ::"r"(CT + 32) : "memory");     // the borrowed stage may be loaded
    const uint32_t a_stage = smem_u32(stage0);
    // Rows of the instruction -> rows of the tile: lanes 0-15 (the half of a warp an 8-byte read is served by at a time)
    // hold instruction rows 0-3, which are the first rows of the tile's first four pairs -- 8 banks apart, all 32 banks
    // between them; lanes 16-31 the pairs' second rows.  (Instruction row = tile row put a pair's two rows, which lie
    // a multiple of 32 banks apart, into the same half: every read took four passes instead of two.)
    const int trow = 2 * (gid & 3) + (gid >> 2);
    const uint32_t o_w = (uint32_t)(gid & 3) * job.w_stride + (gid >> 2) * w_bytes + tig * 8 + g0 * 32, o_s = 8u * job.w_stride + (uint32_t)trow * s_bytes + g0 * 2;
    const uint32_t d_w = 4u * job.w_stride, d_s = 8u * s_bytes, d_b = 16u * s_bytes;
    for (int it = 0; it < my_tiles; it++) {
        const int st = it % S;
        mbar_wait_hot(&full[st], (it / S) & 1, &s_abort, job.status, QW_ST_TMA_TIMEOUT);
        const uint32_t a_w = a_stage + (uint32_t)st * stage_bytes + o_w, a_s = a_stage + (uint32_t)st * stage_bytes + o_s;
        const uint4 sv0 = lds_u4(a_s), sv1 = lds_u4(a_s + d_s), bv0 = lds_u4(a_s + d_b), bv1 = lds_u4(a_s + d_b + d_s);
        const uint32_t s0w[4] = {sv0.x, sv0.y, sv0.z, sv0.w}, s1w[4] = {sv1.x, sv1.y, sv1.z, sv1.w};
        const uint32_t b0w[4] = {bv0.x, bv0.y, bv0.z, bv0.w}, b1w[4] = {bv1.x, bv1.y, bv1.z, bv1.w};
        float ya0[NB], ya1[NB], yb0 = 0.0f, yb1 = 0.0f;        // rows trow, trow + 8: column-pair sums per block, bias sums (token tig)
#pragma unroll
        for (int u = 0; u < NB; u++) { ya0[u] = 0.0f; ya1[u] = 0.0f; }
#pragma unroll
        for (int i = 0; i < QI_PER; i++) {
            const uint2 wa = lds_u2(a_w + 32 * i), wb = lds_u2(a_w + d_w + 32 * i);
            const uint32_t a0 = wa.x & 0x0F0F0F0Fu, a1 = wb.x & 0x0F0F0F0Fu, a2 = (wa.x >> 4) & 0x0F0F0F0Fu, a3 = (wb.x >> 4) & 0x0F0F0F0Fu;
            const uint32_t e0 = wa.y & 0x0F0F0F0Fu, e1 = wb.y & 0x0F0F0F0Fu, e2 = (wa.y >> 4) & 0x0F0F0F0Fu, e3 = (wb.y >> 4) & 0x0F0F0F0Fu;
            int c[NB][4];
#pragma unroll
            for (int u = 0; u < NB; u++) {
                c[u][0] = c[u][1] = c[u][2] = c[u][3] = 0;
                mma_u8s8(c[u], a0, a1, a2, a3, bx[i][u][0].x, bx[i][u][0].y);
                mma_u8s8(c[u], e0, e1, e2, e3, bx[i][u][1].x, bx[i][u][1].y);
            }
            // bf16 pairs: the even group's value is the low half of its word
            const float s_0 = __uint_as_float((i & 1) ? s0w[i >> 1] & 0xffff0000u : s0w[i >> 1] << 16);
            const float s_1 = __uint_as_float((i & 1) ? s1w[i >> 1] & 0xffff0000u : s1w[i >> 1] << 16);
            const float b_0 = __uint_as_float((i & 1) ? b0w[i >> 1] & 0xffff0000u : b0w[i >> 1] << 16);
            const float b_1 = __uint_as_float((i & 1) ? b1w[i >> 1] & 0xffff0000u : b1w[i >> 1] << 16);
            // columns 2 tig, 2 tig + 1 of block u are digits (0, 1) or (2, 3) of token 2 u + tig / 2
#pragma unroll
            for (int u = 0; u < NB; u++) {
                ya0[u] = fmaf(s_0, (float)(c[u][0] + (c[u][1] << 8)), ya0[u]);
                ya1[u] = fmaf(s_1, (float)(c[u][2] + (c[u][3] << 8)), ya1[u]);
            }
            yb0 = fmaf(b_0, xsum[i], yb0);
            yb1 = fmaf(b_1, xsum[i], yb1);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);                 // done with the staged tile
        const int slot = it % QI_SLOTS;
        if (it >= QI_SLOTS) mbar_wait_hot(&pfree[slot], ((it / QI_SLOTS) - 1) & 1, &s_abort, job.status, QW_ST_SLOT_TIMEOUT);
        float *pp = part + (size_t)(slot * W + warp) * 64 * NB, *pq = pbias + (size_t)(slot * W + warp) * 64;
#pragma unroll
        for (int u = 0; u < NB; u++) { pp[trow * 4 * NB + u * 4 + tig] = ya0[u]; pp[(trow + 8) * 4 * NB + u * 4 + tig] = ya1[u]; }
        pq[trow * 4 + tig] = yb0; pq[(trow + 8) * 4 + tig] = yb1;
        __syncwarp();
        if (lane == 0) mbar_arrive(&done[slot]);                // partial sums are in place
    }
}

}  // namespace

// The tensor-path kernel's launch, or false where it does not apply (then the callers below use the
// fp32 kernels): up to four tokens (three and four on the two-instruction form, which takes k up to
// 6144), groups of 64, k a multiple of 512 (so that a row of scales is a whole number of 16-byte
// units), 16-byte aligned operands, at least two tiles staged beside the quantised x in shared memory.
static bool qmv_imma_applies(int k, int group) { return g_tune_qmv_tc && group == 64 && k > 0 && (k & 511) == 0 && k / 512 <= QI_MAXW && k / 8 <= QQ_THREADS * QQ_ITEMS; }
static unsigned qmv_blob_bytes(int k) { return (128u * (unsigned)(k / 8 + 4) + 16u * (unsigned)(k / 64) + 16u + 127u) & ~127u; }
size_t qmv_scratch_bytes(int rows, int k, int group) {
    return rows >= 1 && rows <= 15 && qmv_imma_applies(k, group) ? (size_t)((rows + 3) / 4) * qmv_blob_bytes(k) : 0;
}
// The digits of all rows of x into `blobs` (qmv_scratch_bytes of them), ahead of the products that read them.
static bool launch_qmv_quant(cudaStream_t s, const float *x, void *blobs, int rows, int k) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(4 * ((rows + 3) / 4)); cfg.blockDim = dim3(QQ_THREADS); cfg.dynamicSmemBytes = 0; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_tune_pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, qmv_quant_x_kernel, x, (unsigned char *)blobs, rows, k, qmv_blob_bytes(k)) != cudaSuccess) return false;
    g_launches++;
    return true;
}
static bool launch_qmv_imma(cudaStream_t s, QmvJob &job, int group) {
    const int k = job.k;
    if (!g_tune_qmv_tc || job.tokens < 1 || job.tokens > 4 || group != 64 || k <= 0 || (k & 511)) return false;
    uintptr_t align = reinterpret_cast<uintptr_t>(job.x);
    job.tiles = 0;
    for (int i = 0; i < job.count; i++) {
        if (job.n[i] <= 0) return false;
        align |= reinterpret_cast<uintptr_t>(job.w[i]) | reinterpret_cast<uintptr_t>(job.scales[i]) | reinterpret_cast<uintptr_t>(job.biases[i]);
        job.tiles += (job.n[i] + 15) / 16;
        job.tile_end[i] = job.tiles;
    }
    if (align & 15) return false;
    const int groups = k / group;
    job.per = QI_PER;
    const int W = groups / QI_PER;                              // (k is a multiple of 512)
    const int nb = job.tokens > 2 ? 2 : 1;
    if (W > (nb == 2 ? QI_MAXW4 : QI_MAXW)) return false;
    // staged pairs of rows start 8 banks apart
    int w_words = k / 4; w_words += ((8 - w_words % 32) + 32) % 32;
    job.w_stride = w_words * 4;
    const size_t fixed = (((size_t)groups * 16 + 16 + (size_t)W * 64 * 4 * (nb + 1) * QI_SLOTS + 127) & ~(size_t)127) + 128;
    const size_t stage = 8 * (size_t)job.w_stride + 32 * (size_t)groups * 2, cap = 226 * 1024;
    if (fixed + (nb + 1) * stage > cap) return false;           // (the quantised x borrows nb stages)
    job.stages = (int)std::min<size_t>(QI_MAXS, (cap - fixed) / stage);
    const size_t smem = fixed + job.stages * stage;
    static bool configured[16] = {false};                       // per device
    int dev = 0; cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) return false;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(qmv_imma_q4_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap) != cudaSuccess ||
            cudaFuncSetAttribute(qmv_imma_q4_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap) != cudaSuccess ||
            cudaFuncSetAttribute(qmv_imma_q4_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap) != cudaSuccess ||
            cudaFuncSetAttribute(qmv_imma_q4_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap) != cudaSuccess) return false;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(std::min(job.tiles, sm_count())); cfg.blockDim = dim3((W + 2) * 32); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_tune_pdl ? 1 : 0;
    auto kernel = job.xq ? (nb == 2 ? qmv_imma_q4_kernel<2, true> : qmv_imma_q4_kernel<1, true>)
                         : (nb == 2 ? qmv_imma_q4_kernel<2, false> : qmv_imma_q4_kernel<1, false>);
    if (cudaLaunchKernelEx(&cfg, kernel, job) != cudaSuccess) return false;
    g_launches++;
    return true;
}

void launch_qmv_q4_multi(cudaStream_t s, QmvMulti m, int *status, void *xq) {
    {
        QmvJob job{};
        if (xq && g_tune_qmv_pre == 2 && qmv_scratch_bytes(1, m.k, m.group) && launch_qmv_quant(s, m.x, xq, 1, m.k)) job.xq = (const unsigned char *)xq;
        for (int i = 0; i < m.count; i++) { job.y[i] = m.y[i]; job.w[i] = m.w[i]; job.scales[i] = m.scales[i]; job.biases[i] = m.biases[i]; job.n[i] = m.n[i]; }
        job.x = m.x; job.count = m.count; job.k = m.k; job.tokens = 1; job.status = status;
        if (m.count >= 1 && launch_qmv_imma(s, job, m.group)) return;
    }
    int total = 0;
    for (int i = 0; i < m.count; i++) { m.blocks[i] = (m.n[i] + 8 * QV_OUTS - 1) / (8 * QV_OUTS); total += m.blocks[i]; }
    if (total <= 0) return;
    qmv_q4_multi_kernel<<<total, 256, 0, s>>>(m);
    g_launches++;
}

void launch_qmat_q4(cudaStream_t s, float *y, const float *x, const uint32_t *w, const uint16_t *scales, const uint16_t *biases, int k,
                    int n, int rows, int group, int *status, void *xq) {
    if (n <= 0 || rows <= 0) return;
    // Up to four tokens: the integer tensor kernel, once.  Five to fifteen (the rows of a speculative verify; from 16 on
    // the caller takes the tcgen05 GEMM): the same kernel once per four tokens (per pair where k is beyond the
    // four-token form) -- the weights are streamed once per launch, which is still a fraction of the fp32 kernel's
    // time at these row counts.
    if (rows <= 15) {
        int done = 0, chunk = 4;
        if (xq && !((rows >= 3 ? g_tune_qmv_pre >= 1 : g_tune_qmv_pre == 2) && qmv_scratch_bytes(rows, k, group) && k / 512 <= (rows > 2 ? QI_MAXW4 : QI_MAXW) && launch_qmv_quant(s, x, xq, rows, k)))
            xq = nullptr;
        while (done < rows) {
            QmvJob job{};
            if (xq) job.xq = (const unsigned char *)xq + (size_t)(done / 4) * qmv_blob_bytes(k);
            job.y[0] = y + (size_t)done * n; job.w[0] = w; job.scales[0] = scales; job.biases[0] = biases; job.n[0] = n;
            job.x = x + (size_t)done * k; job.count = 1; job.k = k; job.tokens = std::min(chunk, rows - done); job.status = status;
            if (!launch_qmv_imma(s, job, group)) {
                if (chunk == 4 && job.tokens > 2) { chunk = 2; xq = nullptr; continue; }   // (pairs cut their own digits)
                break;                                           // (the shape does not apply: the kernels below take all rows)
            }
            done += job.tokens;
        }
        if (done == rows) return;
    }
    if (rows <= QV_ROWS && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
        qmv_q4_kernel<<<dim3((n + 8 * QV_OUTS - 1) / (8 * QV_OUTS), 1), 256, 0, s>>>(y, x, w, scales, biases, k, n, rows, group);
        g_launches++;
        return;
    }
    qmat_q4_kernel<<<dim3((n + 7) / 8, (rows + QM_ROWS - 1) / QM_ROWS), 256, 0, s>>>(y, x, w, scales, biases, k, n, rows, group);
    g_launches++;
}

}  // namespace qw
