// Shared device-side helpers for the attention kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda.h>
#include <stdint.h>

#define QW_HEAD_DIM 256          // the only head width the reference builds for (qwasar_metal.m:1359-1363)
#define QW_PAGE_TOKENS 64        // tokens per arena page: 64 x 512 B = 32 KB, 128 B-aligned rows
#define QW_MAX_SEQ 64            // sequences (or row chunks) one launch carries
#define QW_XCHG_REC 264          // floats per exchanged partial: acc[256], max, sum, padding to 16 bytes
#define QW_MAX_MAPS 8            // distinct cache tensor maps one launch carries (arenas of one pool share theirs)

// Status codes a kernel leaves in the backend's status word (first one wins).
enum : int {
    QW_ST_OK = 0,
    QW_ST_TMA_TIMEOUT = 1,       // a wait on a TMA "full" barrier ran out
    QW_ST_SLOT_TIMEOUT = 2,      // a wait on an "empty" barrier ran out
    QW_ST_MMA_TIMEOUT = 3,       // a wait on a tcgen05 commit barrier ran out
    QW_ST_BAD_PAGE = 4,          // a page-table entry was unmapped where a key was needed
    QW_ST_BAD_SMEM = 5,          // the dynamic shared-memory window was not 1024-byte aligned
    QW_ST_PEER_TIMEOUT = 6,      // a partial from another GPU did not arrive within the exchange's time limit
};

namespace qw {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// The status word lives in page-locked host memory mapped into the device: a plain store
// (no atomics across the bus); the first code is kept unless two arrive at once.
__device__ __forceinline__ void report(int *status, int code) {
    volatile int *s = status;
    if (s && *s == 0) *s = code;
}

// ---- programmatic dependent launch -----------------------------------------------
// Kernels of one stream that are launched with the programmatic-serialization attribute may
// start while the kernel before them still runs.  The rules every such kernel here keeps:
//   * nothing produced by the kernel directly before it is read, and nothing any earlier
//     kernel may still read is written, before pdl_wait() has returned (it returns when all
//     earlier kernels have completed and their writes are visible);
//   * pdl_launch_next() is called only after this kernel's own pdl_wait() where the next kernel
//     reads anything before its wait -- so what that kernel finds on starting is at least
//     everything that was complete before this one;
//   * every CTA calls pdl_wait() before it exits, so "this kernel has completed" always implies
//     "every kernel before it has completed".
// Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- mbarrier -----------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Non-blocking probe (try_wait may suspend the thread for a hardware time slice; this never does).
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (seconds), records `code`, raises the
// CTA-wide abort flag so that every later wait returns at once, and returns false.
// Control flow never depends on the outcome, so all warps still meet at the same
// named barriers and the kernel ends.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          int *status, int code) {
    if (*abort_flag) return false;
    for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
        if (mbar_try(bar, parity)) return true;
        if (spin > 64) __nanosleep(spin > 4096 ? 256 : 32);
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    report(status, code);
    return false;
}

// The same bounded wait for hand-offs on a critical path: polls with test_wait first (try_wait
// may park the thread, and waking it costs more than the hand-off it waits for) and looks at
// the abort flag only on the slow path -- under load every shared-memory round trip of the
// waiting thread costs a hundred clocks or more.
__device__ __forceinline__ bool mbar_wait_hot(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                              int *status, int code) {
#pragma unroll 1
    for (uint32_t spin = 0; spin < 4096; ++spin)
        if (mbar_test(bar, parity)) return true;
    return mbar_wait(bar, parity, abort_flag, status, code);
}

// ---- TMA (tiled, no multicast anywhere in this library) -------------------------
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int32_t x, int32_t y,
                                            uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// Tile store, shared -> global, as one bulk group per call site (commit and wait separately).
// Rows or columns of the box that fall outside the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int32_t x, int32_t y, const void *smem_src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// returns once the committed stores have finished reading shared memory
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// Generic-proxy writes to shared memory made visible to the async proxy (TMA / tcgen05).
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- warp-level tensor ops (m16n8k16, bf16 in, fp32 accumulate) ----------------------
__device__ __forceinline__ void ldsm_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// Byte offset of element (row, col) inside one 128B-swizzled box whose rows are 64
// bf16 (128 B) wide; the box base is 1024 B-aligned.  16-byte chunk c of row r sits
// at chunk c ^ (r & 7) -- the layout TMA's SWIZZLE_128B writes.
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t col) {
    return row * 128u + ((((col >> 3) ^ row) & 7u) << 4) + ((col & 7u) << 1);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace qw
