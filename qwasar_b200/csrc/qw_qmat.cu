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

}  // namespace

void launch_qmat_q4(cudaStream_t s, float *y, const float *x, const uint32_t *w, const uint16_t *scales, const uint16_t *biases, int k,
                    int n, int rows, int group) {
    if (n <= 0 || rows <= 0) return;
    qmat_q4_kernel<<<dim3((n + 7) / 8, (rows + QM_ROWS - 1) / QM_ROWS), 256, 0, s>>>(y, x, w, scales, biases, k, n, rows, group);
    g_launches++;
}

}  // namespace qw
