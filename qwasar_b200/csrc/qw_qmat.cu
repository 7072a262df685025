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

// One token, the weights streamed once: x lives in REGISTERS.  A block of W warps splits k: lane l of
// warp w owns the 32-element slots (i * W + w) * 32 + l, i < NS (one 16-byte weight load per slot and
// output row), and keeps those slots' inputs -- and their sums, so that scale and bias come out of
// the inner product -- for every output row it walks.  Blocks are persistent: as many as fit the
// GPU, each striding over chunks of OUTS output rows with the next chunk's weights already on their
// way while the current one is multiplied, so x is fetched once per block and a row costs a lane one
// load and 32 multiply-adds per slot with no shared-memory traffic.
//
// A nibble n becomes a float in ONE instruction: a byte permute drops it into mantissa bits 16-19
// of 0.5f, which is 0.5 (1 + n / 128) exactly; sum_e f_e x_e = 0.5 sum x + (1 / 256) sum n_e x_e, so
// with the slot's sum of x kept beside it the affine weights fold into two multiply-adds per slot:
// y += (256 s) S + (b - 128 s) sum x.  (The products f x are rounded to 24 bits against a signal of
// n x / 256: 1e-6 of a term each, random, far inside the reference's 2e-6 of the sum of absolute
// terms.)  The kernel this replaces staged x in shared memory, read it back twice per weight word,
// converted every nibble through the integer-to-float unit: 7 instructions per weight, a third of
// the warp slots filled, 0.17 of the memory bandwidth.
__device__ __forceinline__ float nib_f(uint32_t bytes, uint32_t sel) {
    // byte `sel & 7` of `bytes` into byte 2 of 0x3F000000
    return __uint_as_float(__byte_perm(bytes, 0x3F000000u, sel));
}
template <int NS, int OUTS>
__global__ void __launch_bounds__(256) qmv1_q4_kernel(float *__restrict__ y, const float *__restrict__ x, const uint32_t *__restrict__ w,
                                                      const uint16_t *__restrict__ scales, const uint16_t *__restrict__ biases, int k,
                                                      int n, int group) {
    __shared__ float part[2][8][OUTS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = blockDim.x >> 5;
    const int words = k >> 3, groups = k / group;
    float xv[NS][32], xsum[NS];
    int slot[NS];
#pragma unroll
    for (int i = 0; i < NS; i++) {
        slot[i] = (i * W + warp) * 32 + lane;
        const bool ok = slot[i] * 32 < k;
        float sum = 0.0f;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const float4 a = ok ? __ldg(reinterpret_cast<const float4 *>(x + (size_t)slot[i] * 32) + u) : make_float4(0.f, 0.f, 0.f, 0.f);
            xv[i][4 * u] = a.x; xv[i][4 * u + 1] = a.y; xv[i][4 * u + 2] = a.z; xv[i][4 * u + 3] = a.w;
            sum += (a.x + a.y) + (a.z + a.w);
        }
        xsum[i] = sum;
        if (!ok) slot[i] = -1;
    }
    const int n_chunks = (n + OUTS - 1) / OUTS;
    uint4 wv[OUTS][NS];
    uint32_t sb[OUTS][NS];                                    // scale (low half) and bias (high half), bf16 bits
    auto fetch = [&](int chunk) {
#pragma unroll
        for (int j = 0; j < OUTS; j++)
#pragma unroll
            for (int i = 0; i < NS; i++) {
                wv[j][i] = make_uint4(0, 0, 0, 0); sb[j][i] = 0u;
                const int o = chunk * OUTS + j;
                if (chunk < n_chunks && o < n && slot[i] >= 0) {
                    wv[j][i] = __ldg(reinterpret_cast<const uint4 *>(w + (size_t)o * words) + slot[i]);
                    const int gi = slot[i] * 32 / group;
                    sb[j][i] = (uint32_t)__ldg(scales + (size_t)o * groups + gi) | ((uint32_t)__ldg(biases + (size_t)o * groups + gi) << 16);
                }
            }
    };
    int chunk = blockIdx.x, it = 0;
    fetch(chunk);
    for (; chunk < n_chunks; chunk += gridDim.x, it++) {
        uint4 cur[OUTS][NS];
        uint32_t csb[OUTS][NS];
#pragma unroll
        for (int j = 0; j < OUTS; j++)
#pragma unroll
            for (int i = 0; i < NS; i++) { cur[j][i] = wv[j][i]; csb[j][i] = sb[j][i]; }
        fetch(chunk + gridDim.x);                               // the next chunk travels under this one's arithmetic
#pragma unroll
        for (int j = 0; j < OUTS; j++) {
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < NS; i++) {
                const uint32_t ww[4] = {cur[j][i].x, cur[j][i].y, cur[j][i].z, cur[j][i].w};
                float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    // nibbles 0, 2, 4, 6 of the word as the four bytes of lo; 1, 3, 5, 7 as those of hi
                    const uint32_t lo = ww[u] & 0x0F0F0F0Fu, hi = (ww[u] >> 4) & 0x0F0F0F0Fu;
                    s1 = fmaf(nib_f(lo, 0x7044), xv[i][8 * u], s1);
                    s2 = fmaf(nib_f(hi, 0x7044), xv[i][8 * u + 1], s2);
                    s1 = fmaf(nib_f(lo, 0x7144), xv[i][8 * u + 2], s1);
                    s2 = fmaf(nib_f(hi, 0x7144), xv[i][8 * u + 3], s2);
                    s1 = fmaf(nib_f(lo, 0x7244), xv[i][8 * u + 4], s1);
                    s2 = fmaf(nib_f(hi, 0x7244), xv[i][8 * u + 5], s2);
                    s1 = fmaf(nib_f(lo, 0x7344), xv[i][8 * u + 6], s1);
                    s2 = fmaf(nib_f(hi, 0x7344), xv[i][8 * u + 7], s2);
                }
                const float sc = __uint_as_float(csb[j][i] << 16), bi = __uint_as_float(csb[j][i] & 0xffff0000u);
                acc = fmaf(256.0f * sc, s1 + s2, acc);
                acc = fmaf(fmaf(-128.0f, sc, bi), xsum[i], acc);
            }
            acc = warp_sum(acc);
            if (lane == 0) part[it & 1][warp][j] = acc;
        }
        __syncthreads();                                        // (the other half of `part` is written next round)
        if (threadIdx.x < OUTS && chunk * OUTS + threadIdx.x < n) {
            float t = 0.0f;
            for (int q = 0; q < W; q++) t += part[it & 1][q][threadIdx.x];
            y[chunk * OUTS + threadIdx.x] = t;
        }
    }
}

}  // namespace

void launch_qmv_q4_multi(cudaStream_t s, QmvMulti m) {
    int total = 0;
    for (int i = 0; i < m.count; i++) { m.blocks[i] = (m.n[i] + 8 * QV_OUTS - 1) / (8 * QV_OUTS); total += m.blocks[i]; }
    if (total <= 0) return;
    qmv_q4_multi_kernel<<<total, 256, 0, s>>>(m);
    g_launches++;
}

void launch_qmat_q4(cudaStream_t s, float *y, const float *x, const uint32_t *w, const uint16_t *scales, const uint16_t *biases, int k,
                    int n, int rows, int group) {
    if (n <= 0 || rows <= 0) return;
    if (rows == 1 && k <= 16384 && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15) == 0 && g_tune_qmv_regs) {
        // one token: the register kernel; W warps so that a lane owns one slot (two for long rows)
        const int slots = k / 32;
        static int per_sm[2][9] = {{0}};                       // resident blocks per SM by (form, warps)
        const int form = slots <= 256 ? 0 : 1, W = form == 0 ? (slots + 31) / 32 : (slots + 63) / 64;
        if (!per_sm[form][W]) {
            int nb = 0;
            if (form == 0) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, qmv1_q4_kernel<1, 4>, W * 32, 0);
            else cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, qmv1_q4_kernel<2, 2>, W * 32, 0);
            per_sm[form][W] = nb > 0 ? nb : 1;
        }
        const int outs = form == 0 ? 4 : 2;
        const int grid = std::min((n + outs - 1) / outs, sm_count() * per_sm[form][W]);
        if (form == 0) qmv1_q4_kernel<1, 4><<<grid, W * 32, 0, s>>>(y, x, w, scales, biases, k, n, group);
        else qmv1_q4_kernel<2, 2><<<grid, W * 32, 0, s>>>(y, x, w, scales, biases, k, n, group);
        g_launches++;
        return;
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
