// The 4-bit affine product for MANY tokens (prefill-side projections, qwasar_gpu.h:116-135) on the
// 5th-generation tensor cores: y[r][o] = sum_i (scale * nibble + bias) * x[r][i] as a GEMM
// Y[rows, n] = X[rows, k] * W^T with the weights dequantised to fp16 in shared memory on their way
// to the tensor core -- the shape of the reference's tensor form (metal4/qmm_tensor.metal:78-260:
// weight tiles unpacked to half in threadgroup memory, x staged as half, the next K step's loads in
// flight during this step's matmul).  Operands are fp16, accumulation fp32; the reference bounds
// that form at 5e-5 of the sum of absolute terms (tests/test_qmv.c:117-131).
//
// One persistent CTA per SM walks tiles of 256 tokens x 256 weight rows (two 128-token halves that share
// every dequantised weight tile: the dequantisation costs as many issue slots per weight as the tensor
// core spends clocks on it at 128 tokens, and a 128 x 256 tile pulled 94 bytes per clock from L2 -- with
// both halves one stage of weights feeds twice the arithmetic); K advances one quantisation group (64)
// per step.  Roles, 14 warps:
//   warp 0      TMA: the step's two X tiles (fp16, 128 x 64 each, SWIZZLE_128B), its 256 x 32 bytes of packed
//               weights, and every eighth step the next 8 groups' scales and biases of the 256 rows
//   warps 2-9   dequantisation, a thread per weight row: 8 packed words -> 64 fp16 = scale * nibble +
//               bias (one fused multiply-add in half2, one rounding), written as the tensor core's
//               K-major SWIZZLE_128B tile; a packed word yields its nibbles in the order 0 4 1 5 2 6 3 7
//               (two masks instead of eight shifts), and X is laid out in that same order by the
//               conversion pass, so no lane ever permutes anything
//   warp 1      one thread issues 8 tcgen05.mma (M128 N256 K16, A and B from shared memory, D in tensor
//               memory) per step and commits the stage back to the producer and the weight buffer back
//               to the dequantisers
//   warps 10-13 epilogue: tensor memory -> registers -> y (fp32); the 512 TMEM columns hold the two
//               halves' 128 x 256 fp32 accumulators, so the epilogue of a tile (a twelfth of its K loop)
//               is not overlapped
// Every mbarrier wait is bounded (a timeout raises the CTA's abort flag and reports through the
// command's status word; control flow never depends on it), tensor memory is always released.
#include <algorithm>
#include "qw_kernels.h"

namespace qw {

namespace {

constexpr int GM = 128, GH = 2, GN = 256, GK = 64, G_NS = 3, G_NB = 2;   // GH halves of GM tokens; TMA stages; weight buffers
constexpr int G_AH_BYTES = GM * GK * 2, G_A_BYTES = GH * G_AH_BYTES, G_B_BYTES = GN * GK * 2, G_W_BYTES = GN * (GK / 2), G_S_BYTES = GN * 16;
constexpr int G_OFF_A = 0, G_OFF_B = G_OFF_A + G_NS * G_A_BYTES, G_OFF_W = G_OFF_B + G_NB * G_B_BYTES;
constexpr int G_OFF_S = G_OFF_W + G_NS * G_W_BYTES;           // [2 slots][scales 256 x 16 B | biases 256 x 16 B]
constexpr int G_OFF_BAR = G_OFF_S + 2 * 2 * G_S_BYTES;
constexpr int G_SMEM = G_OFF_BAR + 256;
constexpr int G_THREADS = 14 * 32;
constexpr int G_W_TMA = 0, G_W_MMA = 1, G_W_DEQ0 = 2, G_W_EPI0 = 10;

__device__ __forceinline__ void g_tmem_alloc(uint32_t *slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void g_tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void g_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void g_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void g_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; descriptors as 32-bit halves (only the low one changes between steps)
__device__ __forceinline__ void g_mma_ss(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 ad, bd;\n\tsetp.ne.u32 p, %6, 0;\n\tmov.b64 ad, {%1, %2};\n\tmov.b64 bd, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], ad, bd, %5, p;\n\t}"
        ::"r"(d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void g_tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr) : "memory");
}
__device__ __forceinline__ void g_tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Shared-memory matrix descriptor, K-major SWIZZLE_128B (layout type 2, version 1): rows of 128 bytes, 8-row groups
// 1024 bytes apart.
__device__ __forceinline__ uint32_t g_desc_lo(uint32_t addr) { return ((addr >> 4) & 0x3FFF) | (1u << 16); }
constexpr uint32_t G_DESC_HI = ((1024u >> 4) & 0x3FFF) | (1u << 14) | (2u << 29);
// kind::f16 instruction descriptor: fp32 accumulate (bit 4), fp16 A and B (formats 0), both K-major, N >> 3 at bit 17,
// M >> 4 at bit 24
constexpr uint32_t G_IDESC = (1u << 4) | ((uint32_t)(GN >> 3) << 17) | ((uint32_t)(GM >> 4) << 24);

// x (fp32 [rows, k]) -> fp16 [rows, k] with every 8 consecutive elements in the order 0 4 1 5 2 6 3 7, the order in
// which a packed weight word gives up its nibbles; values beyond the fp16 range are clamped to it
__global__ void __launch_bounds__(256) qgemm_x16_kernel(uint4 *__restrict__ x16, const float *__restrict__ x, size_t chunks) {
    pdl_wait();
    pdl_launch_next();
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (size_t)gridDim.x * blockDim.x) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(x) + 2 * c), b = __ldg(reinterpret_cast<const float4 *>(x) + 2 * c + 1);
        auto h2 = [](float lo, float hi) {
            const __half2 v = __floats2half2_rn(fminf(fmaxf(lo, -65504.0f), 65504.0f), fminf(fmaxf(hi, -65504.0f), 65504.0f));
            return *reinterpret_cast<const uint32_t *>(&v);
        };
        x16[c] = make_uint4(h2(a.x, b.x), h2(a.y, b.y), h2(a.z, b.z), h2(a.w, b.w));
    }
}

__global__ void __launch_bounds__(G_THREADS, 1) qgemm_q4_kernel(const __grid_constant__ QgemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + G_OFF_BAR);
    uint64_t *full_a = bars, *empty = bars + G_NS;                                     // per TMA stage
    uint64_t *deq = bars + 2 * G_NS, *bq_free = deq + G_NB;                            // per weight buffer
    uint64_t *sc_full = bq_free + G_NB, *sc_empty = sc_full + 2;                       // per scale slot
    uint64_t *acc_full = sc_empty + 2, *acc_empty = acc_full + 1;                      // the accumulators
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool smem_ok = (smem_u32(smem) & 1023u) == 0;          // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) {
        *abort_flag = smem_ok ? 0 : 1;
        if (!smem_ok) report(p.status, QW_ST_BAD_SMEM);
        for (int i = 0; i < G_NS; i++) { mbar_init(&full_a[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < G_NB; i++) { mbar_init(&deq[i], 8); mbar_init(&bq_free[i], 1); }
        for (int i = 0; i < 2; i++) { mbar_init(&sc_full[i], 1); mbar_init(&sc_empty[i], 8); }
        mbar_init(acc_full, 1); mbar_init(acc_empty, 4);
        mbar_fence_init();
    }
    if (warp == G_W_MMA) g_tmem_alloc(tmem_slot, 512);
    g_fence_before();
    __syncthreads();
    g_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();                                                   // x16 comes from the kernel in front
    pdl_launch_next();

    const int gh = p.halves;                                      // 128-token halves per tile: 2, or 1 where that fills the SMs better
    const int m_tiles = (p.rows + gh * GM - 1) / (gh * GM), n_tiles = (p.n + GN - 1) / GN, tiles = m_tiles * n_tiles;
    const int KS = p.k / GK;                                      // K steps per tile (a multiple of 8)
    // The list of work: tiles [0, split_from) whole, each later tile as two entries of one half (the launcher splits the
    // tiles of a last, partly filled round over the SMs so that the round costs a half tile's time).
    const int entries = p.split_from + 2 * (tiles - p.split_from);
    const int my_tiles = (int)blockIdx.x < entries ? (entries - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    auto entry = [&](int it, int &m_t, int &n_t, int &h0, int &halves) {
        const int e = blockIdx.x + it * gridDim.x;
        int tile = e;
        h0 = 0;
        if (e >= p.split_from) { const int j = e - p.split_from; tile = p.split_from + (j >> 1); h0 = j & 1; }
        m_t = tile % m_tiles; n_t = tile / m_tiles;
        halves = e >= p.split_from ? 1 : (p.rows - m_t * gh * GM > GM ? gh : 1);   // (a last tile of at most 128 tokens: one half)
    };

    if (warp == G_W_TMA) {
        if (lane == 0 && smem_ok) {
            for (int it = 0; it < my_tiles; it++) {
                int m_t, n_t, h0, halves;
                entry(it, m_t, n_t, h0, halves);
                for (int ks = 0; ks < KS; ks++) {
                    const int g = it * KS + ks, s = g % G_NS;
                    if ((ks & 7) == 0) {
                        const int sg = g >> 3, slot = sg & 1;
                        if (sg >= 2) mbar_wait(&sc_empty[slot], ((sg >> 1) - 1) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
                        mbar_expect_tx(&sc_full[slot], 2 * G_S_BYTES);
                        tma_load_2d(smem + G_OFF_S + slot * 2 * G_S_BYTES, &p.map_s, ks, n_t * GN, &sc_full[slot]);
                        tma_load_2d(smem + G_OFF_S + slot * 2 * G_S_BYTES + G_S_BYTES, &p.map_b, ks, n_t * GN, &sc_full[slot]);
                    }
                    if (g >= G_NS) mbar_wait(&empty[s], ((g / G_NS) - 1) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
                    mbar_expect_tx(&full_a[s], halves * G_AH_BYTES + G_W_BYTES);
                    for (int h = 0; h < halves; h++)
                        tma_load_2d(smem + G_OFF_A + s * G_A_BYTES + h * G_AH_BYTES, &p.map_x, ks * GK, (m_t * gh + h0 + h) * GM, &full_a[s]);
                    tma_load_2d(smem + G_OFF_W + s * G_W_BYTES, &p.map_w, ks * (GK / 8), n_t * GN, &full_a[s]);
                }
            }
        }
    } else if (warp == G_W_MMA) {
        if (lane == 0 && smem_ok) {
            for (int it = 0; it < my_tiles; it++) {
                int m_t, n_t, h0, halves;
                entry(it, m_t, n_t, h0, halves);
                if (it >= 1) mbar_wait(acc_empty, (it - 1) & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);   // the epilogue has read the last tile
                g_fence_after();
                for (int ks = 0; ks < KS; ks++) {
                    const int g = it * KS + ks, s = g % G_NS, bq = g % G_NB;
                    mbar_wait_hot(&full_a[s], (g / G_NS) & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                    mbar_wait_hot(&deq[bq], (g / G_NB) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
                    g_fence_after();
                    const uint32_t b_lo = g_desc_lo(smem_u32(smem + G_OFF_B + bq * G_B_BYTES));
                    for (int h = 0; h < halves; h++) {
                        const uint32_t a_lo = g_desc_lo(smem_u32(smem + G_OFF_A + s * G_A_BYTES + h * G_AH_BYTES));
#pragma unroll
                        for (int kk = 0; kk < GK / 16; kk++)
                            g_mma_ss(tmem + h * GN, a_lo + kk * 2, G_DESC_HI, b_lo + kk * 2, G_DESC_HI, G_IDESC, (ks | kk) ? 1u : 0u);
                    }
                    g_commit(&empty[s]);                          // the stage is free once these have read it,
                    g_commit(&bq_free[bq]);                       // and so is the weight buffer
                }
                g_commit(acc_full);                               // the tile's accumulators are complete
            }
        }
    } else if (warp < G_W_EPI0) {
        // ---- dequantisation: thread t owns weight row t of the tile
        const int t = threadIdx.x - G_W_DEQ0 * 32;
        const uint32_t row_off = (uint32_t)t * 128u, sw = (uint32_t)(t & 7);
        for (int it = 0; it < my_tiles; it++) {
            for (int ks = 0; ks < KS; ks++) {
                const int g = it * KS + ks, s = g % G_NS, bq = g % G_NB, slot = (g >> 3) & 1;
                if ((ks & 7) == 0) mbar_wait(&sc_full[slot], (g >> 4) & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                mbar_wait(&full_a[s], (g / G_NS) & 1, abort_flag, p.status, QW_ST_TMA_TIMEOUT);
                if (g >= G_NB) mbar_wait(&bq_free[bq], ((g / G_NB) - 1) & 1, abort_flag, p.status, QW_ST_SLOT_TIMEOUT);
                const uint16_t sb = *reinterpret_cast<const uint16_t *>(smem + G_OFF_S + slot * 2 * G_S_BYTES + t * 16 + (ks & 7) * 2);
                const uint16_t bb = *reinterpret_cast<const uint16_t *>(smem + G_OFF_S + slot * 2 * G_S_BYTES + G_S_BYTES + t * 16 + (ks & 7) * 2);
                const __half2 sc = __float2half2_rn(bf16_bits_to_f32(sb)), bi = __float2half2_rn(bf16_bits_to_f32(bb));
                const uint4 w0 = *reinterpret_cast<const uint4 *>(smem + G_OFF_W + s * G_W_BYTES + t * 32);
                const uint4 w1 = *reinterpret_cast<const uint4 *>(smem + G_OFF_W + s * G_W_BYTES + t * 32 + 16);
                const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                uint8_t *brow = smem + G_OFF_B + bq * G_B_BYTES + row_off;
                const __half2 k1024 = __float2half2_rn(1024.0f);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    // 0x6400 | nibble is the fp16 number 1024 + nibble: two nibbles per instruction, then minus 1024
                    // (exact) and one fused multiply-add
                    uint32_t h[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const uint32_t bits = ((ww[j] >> (4 * q)) & 0x000F000Fu) | 0x64006400u;
                        const __half2 v = __hfma2(__hsub2(*reinterpret_cast<const __half2 *>(&bits), k1024), sc, bi);
                        h[q] = *reinterpret_cast<const uint32_t *>(&v);
                    }
                    *reinterpret_cast<uint4 *>(brow + (((uint32_t)j ^ sw) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                }
                fence_proxy_async();                              // these writes, before the tensor core's reads
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&deq[bq]);
                    if ((ks & 7) == 7) mbar_arrive(&sc_empty[slot]);
                }
            }
        }
    } else {
        // ---- epilogue: this warp reads the TMEM lanes of its quarter (warp index mod 4), a lane = a token
        const int q = warp & 3;
        for (int it = 0; it < my_tiles; it++) {
            int m_t, n_t, h0, halves;
            entry(it, m_t, n_t, h0, halves);
            mbar_wait(acc_full, it & 1, abort_flag, p.status, QW_ST_MMA_TIMEOUT);
            g_fence_after();
            for (int h = 0; h < halves; h++) {
                const int row = (m_t * gh + h0 + h) * GM + q * 32 + lane;
                float *yrow = p.y + (size_t)row * p.n + (size_t)n_t * GN;
#pragma unroll 1
                for (int c = 0; c < GN / 32; c++) {
                    uint32_t r[32];
                    g_tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + h * GN + c * 32, r);
                    g_tmem_wait_ld();
                    if (row < p.rows && !*abort_flag) {
                        const int col0 = n_t * GN + c * 32;
#pragma unroll
                        for (int v = 0; v < 8; v++)
                            if (col0 + v * 4 < p.n)               // (n is a multiple of 4)
                                *reinterpret_cast<float4 *>(yrow + c * 32 + v * 4) =
                                    make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                    }
                }
            }
            g_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
        }
    }
    g_fence_before();
    __syncthreads();
    if (warp == G_W_MMA) g_tmem_dealloc(tmem, 512);
}

}  // namespace

int g_tune_qmm_tc = 1;

size_t qgemm_scratch_bytes(int rows, int k) { return (size_t)rows * k * 2; }

bool launch_qgemm_q4(cudaStream_t s, const QgemmParams &p, const float *x, void *x16) {
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return false;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(qgemm_q4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM) != cudaSuccess) return false;
        configured[dev] = true;
    }
    const size_t chunks = (size_t)p.rows * p.k / 8;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_tune_pdl ? 1 : 0; cfg.stream = s;
    cfg.gridDim = dim3((unsigned)std::min<size_t>((chunks + 255) / 256, (size_t)sm_count() * 8)); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0;
    if (cudaLaunchKernelEx(&cfg, qgemm_x16_kernel, reinterpret_cast<uint4 *>(x16), x, chunks) != cudaSuccess) return false;
    g_launches++;
    // Two halves per tile cost a step 512 tensor-core clocks, one half about 340 (bound by the dequantisation; measured 730 against 950 TFLOP/s on a large product):
    // whichever gets through its rounds over the SMs sooner
    const int n_tiles = (p.n + GN - 1) / GN, sms = sm_count();
    const int t2 = ((p.rows + 2 * GM - 1) / (2 * GM)) * n_tiles, t1 = ((p.rows + GM - 1) / GM) * n_tiles;
    QgemmParams q = p;
    q.halves = (long long)((t2 + sms - 1) / sms) * 512 <= (long long)((t1 + sms - 1) / sms) * 340 ? 2 : 1;
    int tiles = q.halves == 2 ? t2 : t1;
    q.split_from = tiles;
    if (q.halves == 2 && (p.rows % (2 * GM) == 0 || p.rows % (2 * GM) > GM)) {       // every tile has both halves
        const int rem = tiles % sms;                            // tiles of the last, partly filled round
        if (rem > 0 && 2 * rem <= sms) { q.split_from = tiles - rem; tiles += rem; }
    }
    cfg.gridDim = dim3((unsigned)std::min(tiles, sms)); cfg.blockDim = dim3(G_THREADS); cfg.dynamicSmemBytes = G_SMEM;
    if (cudaLaunchKernelEx(&cfg, qgemm_q4_kernel, q) != cudaSuccess) return false;
    g_launches++;
    return true;
}

}  // namespace qw
