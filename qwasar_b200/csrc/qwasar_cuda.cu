// qwasar_cuda.cu -- the C-ABI CUDA backend for the gated attention path (sm_100a).
//
// The sibling of the reference's qwasar_metal.m for the subset of qwasar_gpu.h that
// the attention node uses: device bring-up, buffers, command buffers (one CUDA
// stream each), the paged K/V arena, and host dispatch of the kernels in
// qw_preops.cu / qw_decode.cu / qw_prefill.cu.  Error convention of the
// reference: void ops encode nothing on a bad argument, bool ops return false
// "encoding nothing", device errors surface as a string from qw_cmd_error after
// qw_cmd_wait.  There is no CPU path: without a CUDA device qw_gpu_init fails
// and every op declines.
#include "../../include/qwasar_cuda.h"
#include "qw_kernels.h"

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

using namespace qw;

// ---------------------------------------------------------------------------------------
// state
// ---------------------------------------------------------------------------------------
namespace {

enum BufKind { BUF_SHARED, BUF_DEVICE, BUF_ARENA, BUF_POOL };

struct Arena;
struct Pool;

}  // namespace

struct qw_buf_s {
    BufKind kind;
    size_t len;
    void *host;          // shared: pinned (or caller's) host memory
    void *dev;           // device side (shared mirror, device buffer, or arena pool)
    bool own_host, own_dev, registered;
    Arena *arena;
    Pool *pool = nullptr;   // BUF_POOL: the page pool this handle stands for
    int device = 0;      // the CUDA device the buffer lives on
};

namespace {

struct Touch {
    qw_buf b;
    size_t lo, hi;       // byte range whose device mirror is current in this command buffer
    size_t wlo, whi;     // hull of the ranges ops wrote (whi == 0: none)
};
struct Scratch { void *p; size_t n; };
struct Mark { cudaEvent_t ev; const char *label; };
struct KTime { cudaEvent_t t0, t1; const char *kernel; };

}  // namespace

struct qw_cmd_s {
    cudaStream_t stream;
    int device = 0;                 // the CUDA device of the stream; ops switch to it before they launch
    int status_slot = 0;            // this command buffer's kernel status word (slot 0 is shared when all are taken)
    bool own_stream;
    bool failed;
    char err[256];
    int parallel;
    std::vector<Touch> touched;
    cudaEvent_t uploaded = nullptr; // last first-touch upload on the copy stream (see dev_range)
    cudaEvent_t written = nullptr, downloaded = nullptr;   // early copy-back at qw_cmd_flush (see there)
    bool early_down = false;
    std::vector<Scratch> scratch;   // last one is current; earlier ones may still be in flight
    std::vector<Mark> marks;
    std::vector<KTime> ktimes;
};

namespace {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*PFN_memAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
typedef CUresult (*PFN_memAddressFree)(CUdeviceptr, size_t);
typedef CUresult (*PFN_memCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
typedef CUresult (*PFN_memRelease)(CUmemGenericAllocationHandle);
typedef CUresult (*PFN_memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
typedef CUresult (*PFN_memUnmap)(CUdeviceptr, size_t);
typedef CUresult (*PFN_memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
typedef CUresult (*PFN_memGetGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);

// One of these per CUDA device (qw_gpu_init brings up the current device, qw_gpu_init_multi
// several); G is the state of the device that is current for this library.
constexpr int MAX_DEVICES = 16;
constexpr int STATUS_SLOTS = 64, STATUS_STRIDE = 16;     // status words, 64 bytes apart
struct Globals {
    bool up = false;
    int device = 0;
    int sms = 0;
    cudaDeviceProp prop;
    char name[300] = "";
    int *status_host = nullptr;    // pinned + mapped: kernels record a status code in their command buffer's word
    int *status_dev = nullptr;
    uint64_t status_used = 1;      // bit i: slot i belongs to a live command buffer (slot 0: the shared one)
    PFN_encodeTiled encodeTiled = nullptr;
    PFN_memAddressReserve memAddressReserve = nullptr;
    PFN_memAddressFree memAddressFree = nullptr;
    PFN_memCreate memCreate = nullptr;
    PFN_memRelease memRelease = nullptr;
    PFN_memMap memMap = nullptr;
    PFN_memUnmap memUnmap = nullptr;
    PFN_memSetAccess memSetAccess = nullptr;
    PFN_memGetGranularity memGetGranularity = nullptr;
    std::vector<Scratch> scratch_pool;
    std::vector<cudaStream_t> stream_pool;    // streams of freed command buffers, reused
    cudaStream_t copy_stream = nullptr;       // first-touch uploads of shared buffers, see dev_range
    cudaStream_t down_stream = nullptr;       // copy-back of written ranges started at qw_cmd_flush
    std::map<std::pair<uintptr_t, uint64_t>, CUtensorMap> map_cache;   // linear caches: (base, rows * 128 + box rows) -> map
};
Globals g_devs[MAX_DEVICES];
Globals *g_cur = &g_devs[0];
#define G (*g_cur)

// Process-wide: the last error of a call without a command buffer, and the profiling tables.
struct Shared {
    char last_error[256] = "";
    bool has_error = false;
    int prof = -1;
    std::map<std::string, std::pair<double, long>> prof_ms;
    bool time_kernels = false;
    std::map<std::string, std::pair<double, long long>> kernel_ms;
} SH;

// Makes `dev` the current device of this library and of the calling thread.
void use_device(int dev) {
    if (dev < 0 || dev >= MAX_DEVICES || g_cur == &g_devs[dev]) return;
    cudaSetDevice(dev);
    g_cur = &g_devs[dev];
}

int *cmd_status(qw_cmd c) { return G.status_dev + (size_t)c->status_slot * STATUS_STRIDE; }

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(SH.last_error, sizeof SH.last_error, fmt, ap);
    va_end(ap);
    SH.has_error = true;
}

void cmd_fail(qw_cmd c, const char *fmt, ...) {
    if (!c || c->failed) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(c->err, sizeof c->err, fmt, ap);
    va_end(ap);
    c->failed = true;
}

bool cuda_ok(qw_cmd c, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return true;
    cmd_fail(c, "%s: %s", what, cudaGetErrorString(e));
    return false;
}

template <typename T>
bool entry(const char *name, T *fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
        return false;
    *fn = reinterpret_cast<T>(p);
    return true;
}

const char *status_text(int code) {
    switch (code) {
        case QW_ST_TMA_TIMEOUT: return "kernel gave up waiting for a TMA load";
        case QW_ST_SLOT_TIMEOUT: return "kernel gave up waiting for a free pipeline stage";
        case QW_ST_MMA_TIMEOUT: return "kernel gave up waiting for a tensor-core commit";
        case QW_ST_BAD_PAGE: return "attention reached a cache position whose page was never mapped";
        case QW_ST_BAD_SMEM: return "the prefill kernel's shared-memory window was not 1024-byte aligned";
        case QW_ST_PEER_TIMEOUT: return "the partial of another GPU did not arrive within the exchange's time limit";
        default: return "unknown kernel status";
    }
}

// ---------------------------------------------------------------------------------------
// the paged arena
// ---------------------------------------------------------------------------------------
constexpr size_t PAGE_BYTES = (size_t)QW_PAGE_TOKENS * QW_HEAD_DIM * 2;   // 32 KB
constexpr size_t CHUNK_BYTES = (size_t)64 << 20;                           // physical growth step
constexpr int PAGES_PER_CHUNK = (int)(CHUNK_BYTES / PAGE_BYTES);

// A pool is a reserved range of device addresses that fills with 32 KB pages as tokens arrive;
// arenas (one per cache buffer of the reference) draw their pages from a pool.  Arenas that share
// a pool share its tensor maps, so one attention launch can carry any number of their sequences.
struct Pool {
    int device;
    bool vmm;
    CUdeviceptr va;
    size_t va_size;
    std::vector<CUmemGenericAllocationHandle> chunks;
    int64_t max_pages;
    int64_t mapped_pages;                 // pool pages backed by physical memory
    std::vector<int32_t> free_pages;
    uint32_t shuffle;
    int refs;                             // arenas (and the pool's own handle) that keep it alive
    CUtensorMap map;                      // 32-row boxes (split-KV kernel)
    CUtensorMap map64;                    // 64-row boxes (prefill kernel)
};
struct Arena {
    Pool *pool;
    int n_layers, kv_heads, max_ctx, head_dim;
    int pages_per_head;
    int64_t max_pages;
    std::vector<int32_t> table_host;      // [n_layers, kv_heads, pages_per_head], -1 = unmapped
    int32_t *table_dev;
    int64_t in_use;
};

bool encode_rows_map(CUtensorMap *m, void *base, uint64_t rows, uint32_t box_rows) {
    cuuint64_t dims[2] = {QW_HEAD_DIM, rows};
    cuuint64_t strides[1] = {QW_HEAD_DIM * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = G.encodeTiled(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return false; }
    return true;
}

// A [rows][row_elems] tensor of bf16 or f32 with a row pitch of pitch_elems, as 128-byte x 128-row boxes.
bool encode_tile_map(CUtensorMap *m, const void *base, int dtype, uint64_t row_elems, uint64_t pitch_elems, uint64_t rows) {
    const uint32_t el = dtype == DT_BF16 ? 2 : 4;
    cuuint64_t dims[2] = {row_elems, rows};
    cuuint64_t strides[1] = {pitch_elems * el};
    cuuint32_t box[2] = {128 / el, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = G.encodeTiled(m, dtype == DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                               const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return false; }
    return true;
}

// A row-major 2-D tensor [rows][inner] of el-byte elements with a row pitch in bytes, as boxes of box_inner x box_rows.
bool encode_2d_map(CUtensorMap *m, const void *base, CUtensorMapDataType type, uint32_t el, uint64_t inner, uint64_t pitch_bytes,
                   uint64_t rows, uint32_t box_inner, uint32_t box_rows, bool swizzle128) {
    (void)el;
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = G.encodeTiled(m, type, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return false; }
    return true;
}

bool pool_grow(Pool *a) {
    if (a->mapped_pages >= a->max_pages) { set_error("page pool exhausted (%lld pages)", (long long)a->max_pages); return false; }
    const int64_t first = a->mapped_pages;
    const int64_t n = std::min<int64_t>(PAGES_PER_CHUNK, a->max_pages - first);
    if (a->vmm) {
        CUmemAllocationProp prop = {};
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = a->device;
        CUmemGenericAllocationHandle h;
        // the reserved range is a whole number of chunks, so a full chunk is always mapped
        if (G.memCreate(&h, CHUNK_BYTES, &prop, 0) != CUDA_SUCCESS) { set_error("arena: out of device memory"); return false; }
        const CUdeviceptr at = a->va + (size_t)first * PAGE_BYTES;
        if (G.memMap(at, CHUNK_BYTES, 0, h, 0) != CUDA_SUCCESS) { G.memRelease(h); set_error("arena: cuMemMap failed"); return false; }
        CUmemAccessDesc acc = {};
        acc.location = prop.location;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        if (G.memSetAccess(at, CHUNK_BYTES, &acc, 1) != CUDA_SUCCESS) {
            G.memUnmap(at, CHUNK_BYTES); G.memRelease(h); set_error("arena: cuMemSetAccess failed"); return false;
        }
        a->chunks.push_back(h);
        // The new pages start as zeros, and the fill has finished before any stream can be handed
        // one of them: command streams do not order with one another, so a fill left pending on one
        // stream could land on rows that another stream has already appended.  Growth is rare
        // (64 MB steps), so the wait costs nothing that matters.
        if (cudaMemset(reinterpret_cast<void *>(at), 0, CHUNK_BYTES) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
            set_error("arena: clearing a new chunk failed");
            return false;
        }
    }
    // hand the new pages to the free list, permuted when asked to
    std::vector<int32_t> ids((size_t)n);
    for (int64_t i = 0; i < n; i++) ids[(size_t)i] = (int32_t)(first + i);
    if (a->shuffle) {
        uint32_t s = a->shuffle ^ (uint32_t)first ^ 0x9e3779b9u;
        for (int64_t i = n - 1; i > 0; i--) {
            s ^= s << 13; s ^= s >> 17; s ^= s << 5;
            std::swap(ids[(size_t)i], ids[(size_t)(s % (uint32_t)(i + 1))]);
        }
    }
    // free_pages is popped from the back: keep ascending order there when not shuffling
    for (int64_t i = n - 1; i >= 0; i--) a->free_pages.push_back(ids[(size_t)i]);
    a->mapped_pages += n;
    return true;
}

// Makes sure the pages that hold tokens [first_token, n_tokens) of `layer` exist, and pushes new
// page-table entries to the device in stream order.  Pages below first_token are left alone: a
// rank that owns only a range of positions maps only that range.
bool arena_ensure(Arena *a, int layer, int first_token, int n_tokens, cudaStream_t stream) {
    const int need = (n_tokens + QW_PAGE_TOKENS - 1) / QW_PAGE_TOKENS;
    const int first_page = std::max(first_token, 0) / QW_PAGE_TOKENS;
    if (need > a->pages_per_head) { set_error("arena: %d tokens exceed max_ctx %d", n_tokens, a->max_ctx); return false; }
    Pool *pl = a->pool;
    for (int h = 0; h < a->kv_heads; h++) {
        int32_t *row = a->table_host.data() + ((size_t)layer * a->kv_heads + h) * a->pages_per_head;
        int first_new = -1, last_new = -1;
        for (int pg = first_page; pg < need; pg++) {
            if (row[pg] >= 0) continue;
            if (pl->free_pages.empty() && !pool_grow(pl)) return false;
            row[pg] = pl->free_pages.back();
            pl->free_pages.pop_back();
            a->in_use++;
            if (first_new < 0) first_new = pg;
            last_new = pg;
        }
        if (first_new >= 0) {
            const size_t off = ((size_t)layer * a->kv_heads + h) * a->pages_per_head + first_new;
            // pageable source: the runtime stages it before returning, the copy itself is in stream order
            if (cudaMemcpyAsync(a->table_dev + off, a->table_host.data() + off,
                                (size_t)(last_new - first_new + 1) * sizeof(int32_t), cudaMemcpyHostToDevice,
                                stream) != cudaSuccess) {
                set_error("arena: page-table update failed");
                return false;
            }
        }
    }
    return true;
}

void pool_release(Pool *pl) {
    if (!pl || --pl->refs > 0) return;
    use_device(pl->device);
    cudaDeviceSynchronize();
    if (pl->vmm) {
        for (size_t i = 0; i < pl->chunks.size(); i++) {
            G.memUnmap(pl->va + i * CHUNK_BYTES, CHUNK_BYTES);
            G.memRelease(pl->chunks[i]);
        }
        if (pl->va) G.memAddressFree(pl->va, pl->va_size);
    } else if (pl->va) {
        cudaFree(reinterpret_cast<void *>(pl->va));
    }
    delete pl;
}

// A pool able to hold max_bytes of pages (rounded up to whole 64 MB chunks); nothing is committed yet.
Pool *pool_create(size_t max_bytes, uint32_t shuffle) {
    Pool *pl = new Pool();
    pl->device = G.device;
    const size_t n_chunks = std::max<size_t>(1, (max_bytes + CHUNK_BYTES - 1) / CHUNK_BYTES);
    pl->va_size = n_chunks * CHUNK_BYTES;
    pl->max_pages = (int64_t)(pl->va_size / PAGE_BYTES);
    pl->mapped_pages = 0; pl->shuffle = shuffle; pl->refs = 1; pl->va = 0; pl->vmm = false;
    if (G.memAddressReserve) {
        CUmemAllocationProp prop = {};
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = G.device;
        size_t gran = 0;
        if (G.memGetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM) == CUDA_SUCCESS && gran && CHUNK_BYTES % gran == 0 &&
            G.memAddressReserve(&pl->va, pl->va_size, CHUNK_BYTES, 0, 0) == CUDA_SUCCESS)
            pl->vmm = true;
    }
    if (!pl->vmm) {
        // no virtual-memory management on this platform: the pool is allocated whole
        void *p = nullptr;
        if (cudaMalloc(&p, pl->va_size) != cudaSuccess) { set_error("arena: cannot allocate %zu bytes", pl->va_size); delete pl; cudaGetLastError(); return nullptr; }
        cudaMemset(p, 0, pl->va_size);
        cudaDeviceSynchronize();
        pl->va = (CUdeviceptr)p;
        pl->mapped_pages = 0;             // pages still enter the free list chunk by chunk (pool_grow)
    }
    // the tensor maps span the whole reserved range; rows of unmapped pages are never addressed
    if (!encode_rows_map(&pl->map, reinterpret_cast<void *>(pl->va), (uint64_t)(pl->va_size / 512), 32) ||
        !encode_rows_map(&pl->map64, reinterpret_cast<void *>(pl->va), (uint64_t)(pl->va_size / 512), 64)) { pool_release(pl); return nullptr; }
    return pl;
}

void arena_destroy(Arena *a) {
    if (!a) return;
    use_device(a->pool->device);
    cudaDeviceSynchronize();
    // the arena's pages go back to its pool (they keep their contents: an arena that is handed a
    // recycled page owns every row of it only after it has appended that row)
    for (int32_t id : a->table_host) if (id >= 0) a->pool->free_pages.push_back(id);
    if (a->table_dev) cudaFree(a->table_dev);
    pool_release(a->pool);
    delete a;
}

// ---------------------------------------------------------------------------------------
// buffers, coherence of shared buffers, scratch
// ---------------------------------------------------------------------------------------

// Device address of [off, off+bytes) of a ref.  For shared buffers the device mirror of
// that range is brought up to date (once per command buffer) and, when `write`, marked
// for copy-back at qw_cmd_wait.  Activations and weights move as 16-byte pieces: an operand
// that does not start on a 16-byte boundary is refused here (an error string, not a fault);
// the small tables (positions, axes, frequencies) pass their own element size.
void *dev_range(qw_cmd c, qw_ref r, size_t bytes, bool write, size_t align = 16) {
    qw_buf b = r.buf;
    if (!b) return nullptr;
    if (b->kind == BUF_ARENA || b->kind == BUF_POOL) { cmd_fail(c, "an arena can only be a cache operand"); return nullptr; }
    if (r.off + bytes > b->len) { cmd_fail(c, "operand [%zu, %zu) exceeds its buffer (%zu bytes)", r.off, r.off + bytes, b->len); return nullptr; }
    if ((reinterpret_cast<uintptr_t>(b->dev) + r.off) & (align - 1)) {
        cmd_fail(c, "operand at byte offset %zu of its buffer is not %zu-byte aligned", r.off, align);
        return nullptr;
    }
    if (b->kind == BUF_SHARED && bytes) {
        // small buffers are mirrored whole on first touch: one copy instead of one per operand
        const bool whole = b->len <= ((size_t)4 << 20);
        const size_t lo = whole ? 0 : r.off, hi = whole ? b->len : r.off + bytes;
        const size_t w_lo = r.off, w_hi = r.off + bytes;
        Touch *t = nullptr;
        for (auto &x : c->touched) if (x.b == b) { t = &x; break; }
        if (!t) {
            c->touched.push_back(Touch{b, lo, hi, 0, 0});
            t = &c->touched.back();
            // The first upload of a buffer in a command buffer goes to the copy stream and the
            // command's stream waits for it: nothing encoded earlier in this command buffer can
            // have used the mirror, and the caller may not change a buffer that an uncompleted
            // command buffer uses, so the copy may run while the ops encoded before it (the
            // layers before this one) still execute instead of queueing behind them.
            if (!c->uploaded && cudaEventCreateWithFlags(&c->uploaded, cudaEventDisableTiming) != cudaSuccess) c->uploaded = nullptr;
            cudaStream_t up = G.copy_stream && c->uploaded ? G.copy_stream : c->stream;
            cuda_ok(c, cudaMemcpyAsync((char *)b->dev + lo, (char *)b->host + lo, hi - lo, cudaMemcpyHostToDevice, up), "upload");
            if (up != c->stream) {
                cuda_ok(c, cudaEventRecord(c->uploaded, up), "upload event");
                cuda_ok(c, cudaStreamWaitEvent(c->stream, c->uploaded, 0), "upload wait");
            }
        } else {
            if (lo < t->lo) {
                cuda_ok(c, cudaMemcpyAsync((char *)b->dev + lo, (char *)b->host + lo, t->lo - lo, cudaMemcpyHostToDevice, c->stream), "upload");
                t->lo = lo;
            }
            if (hi > t->hi) {
                cuda_ok(c, cudaMemcpyAsync((char *)b->dev + t->hi, (char *)b->host + t->hi, hi - t->hi, cudaMemcpyHostToDevice, c->stream), "upload");
                t->hi = hi;
            }
        }
        if (write) {
            if (t->whi == 0) { t->wlo = w_lo; t->whi = w_hi; }
            else { t->wlo = std::min(t->wlo, w_lo); t->whi = std::max(t->whi, w_hi); }
        }
    }
    return (char *)b->dev + r.off;
}

void *cmd_scratch(qw_cmd c, size_t bytes) {
    bytes = (bytes + 1023) & ~(size_t)1023;
    if (!c->scratch.empty() && c->scratch.back().n >= bytes) return c->scratch.back().p;
    // a block from the pool, else a new allocation (never inside a steady-state step:
    // blocks return to the pool when their command buffer is freed)
    size_t best = (size_t)-1;
    for (size_t i = 0; i < G.scratch_pool.size(); i++)
        if (G.scratch_pool[i].n >= bytes && (best == (size_t)-1 || G.scratch_pool[i].n < G.scratch_pool[best].n)) best = i;
    Scratch s;
    if (best != (size_t)-1) {
        s = G.scratch_pool[best];
        G.scratch_pool.erase(G.scratch_pool.begin() + (long)best);
    } else {
        s.n = std::max(bytes, (size_t)8 << 20);
        if (cudaMalloc(&s.p, s.n) != cudaSuccess) { cmd_fail(c, "cannot allocate %zu bytes of scratch", s.n); return nullptr; }
    }
    c->scratch.push_back(s);
    return s.p;
}

bool shape_ok(int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_ctx, int32_t base_pos) {
    return rows > 0 && kv_heads > 0 && q_heads > 0 && q_heads % kv_heads == 0 && head_dim == QW_HEAD_DIM &&
           base_pos >= 0 && (int64_t)base_pos + rows <= max_ctx;
}

// One layer's cache operand -> KvLayer + tensor map.  n_tokens: positions that must be
// addressable (pages are mapped up to there when `append`).
bool resolve_cache(qw_cmd c, qw_ref ref, int32_t kv_heads, int32_t max_ctx, int32_t head_dim, int32_t n_tokens,
                   bool append, bool will_write, KvLayer *out, CUtensorMap *map, uint32_t box_rows = 32,
                   int64_t *map_rows = nullptr, int32_t first_token = 0) {
    qw_buf b = ref.buf;
    if (!b) { cmd_fail(c, "cache operand is null"); return false; }
    if (b->kind == BUF_POOL) { cmd_fail(c, "a page pool is not a cache: allocate an arena in it"); return false; }
    const size_t layer_bytes = (size_t)kv_heads * max_ctx * head_dim * 2;
    if (b->kind == BUF_ARENA) {
        Arena *a = b->arena;
        if (a->kv_heads != kv_heads || a->max_ctx != max_ctx || a->head_dim != head_dim) {
            cmd_fail(c, "arena was created for [%d heads, %d ctx, %d dim], op says [%d, %d, %d]", a->kv_heads, a->max_ctx,
                     a->head_dim, kv_heads, max_ctx, head_dim);
            return false;
        }
        if (ref.off % layer_bytes) { cmd_fail(c, "arena offset %zu is not a layer boundary", ref.off); return false; }
        const int layer = (int)(ref.off / layer_bytes);
        if (layer >= a->n_layers) { cmd_fail(c, "arena layer %d out of range", layer); return false; }
        if (append && !arena_ensure(a, layer, first_token, n_tokens, c->stream)) { cmd_fail(c, "%s", SH.last_error); return false; }
        out->base = reinterpret_cast<__nv_bfloat16 *>(a->pool->va);
        out->table = a->table_dev + (size_t)layer * a->kv_heads * a->pages_per_head;
        out->pt_stride = a->pages_per_head;
        out->max_ctx = max_ctx;
        if (map) *map = box_rows == 64 ? a->pool->map64 : a->pool->map;
        if (map_rows) *map_rows = (int64_t)(a->pool->va_size / 512);
        return true;
    }
    void *d = dev_range(c, ref, layer_bytes, will_write);
    if (!d) return false;
    if ((uintptr_t)d & 127) { cmd_fail(c, "cache operand is not 128-byte aligned"); return false; }
    out->base = reinterpret_cast<__nv_bfloat16 *>(d);
    out->table = nullptr;
    out->pt_stride = 0;
    out->max_ctx = max_ctx;
    if (map) {
        const uint64_t rows = (uint64_t)kv_heads * max_ctx;
        auto key = std::make_pair((uintptr_t)d, rows * 128 + box_rows);
        auto it = G.map_cache.find(key);
        if (it == G.map_cache.end()) {
            CUtensorMap m;
            if (!encode_rows_map(&m, d, rows, box_rows)) { cmd_fail(c, "%s", SH.last_error); return false; }
            it = G.map_cache.emplace(key, m).first;
        }
        *map = it->second;
        if (map_rows) *map_rows = (int64_t)rows;
    }
    return true;
}

// Fills the schedule fields of a launch's sequences and sizes its grid.
void plan_split(AttnParams &p) {
    int cum = 0;
    int row_slot = 0;
    for (int i = 0; i < p.n_seq; i++) {
        AttnSeq &s = p.seq[i];
        s.tile0 = s.key_lo / 32;
        s.n_tiles = std::max(1, (s.key_hi + 31) / 32 - s.tile0);
        s.cum_tiles = cum;
        s.row_slot0 = row_slot;
        cum += s.n_tiles * p.kv_heads;
        row_slot += s.rows;
    }
    p.total_tiles = cum;
    p.n_cta = std::min(std::min(sm_count(), 256), cum);      // the merge kernel reads one partial per thread of 256
}

// Launches the split-KV kernel (and the merge where any group was cut) for the sequences
// already described in p.seq; `scr` holds attn_split_scratch_bytes(p, max_rows).
bool launch_split_merge(qw_cmd c, AttnParams &p, int max_rows, float *scr) {
    const int mt16 = ((max_rows * p.gqa + 15) / 16 <= 1 ? 1 : ((max_rows * p.gqa + 15) / 16 <= 2 ? 2 : 4)) * 16;
    size_t rows_total = 0;
    for (int i = 0; i < p.n_seq; i++) rows_total += p.seq[i].rows;
    const size_t n_part_rows = (size_t)attn_split_slots(p) * mt16 + rows_total * p.q_heads;
    p.pacc = scr;
    p.pstat = scr + n_part_rows * 256;
    p.status = cmd_status(c);
    KTime kt = {nullptr, nullptr, "qw_attn_split"};
    const bool timed = SH.time_kernels && cudaEventCreate(&kt.t0) == cudaSuccess && cudaEventCreate(&kt.t1) == cudaSuccess;
    if (timed) cudaEventRecord(kt.t0, c->stream);
    launch_attn_split(c->stream, p, max_rows);
    if (timed) { cudaEventRecord(kt.t1, c->stream); c->ktimes.push_back(kt); }
    // a group is written directly only when one CTA's share covers it whole
    if (p.mode != 0 || attn_split_needs_merge(p)) launch_attn_merge(c->stream, p, max_rows);
    return cuda_ok(c, cudaGetLastError(), "attention launch");
}

// Split-KV attention of up to QW_MAX_SEQ sequences already described in p.seq (q, out,
// gate, caches, rows, base_pos, key range).  max_rows * gqa <= 64.
bool run_split(qw_cmd c, AttnParams &p, int max_rows) {
    plan_split(p);
    float *scr = (float *)cmd_scratch(c, attn_split_scratch_bytes(p, max_rows));
    if (!scr) return false;
    return launch_split_merge(c, p, max_rows, scr);
}

// Collects sequences (or row chunks) for split-KV launches: one launch carries up to QW_MAX_SEQ of
// them over up to QW_MAX_MAPS distinct cache tensor maps (arenas of one pool share one map, plain
// cache buffers have one each); a sequence that does not fit starts the next launch.
struct SplitBatch {
    qw_cmd c;
    AttnParams p;
    int n = 0, n_maps = 0, max_rows = 0;
    bool early_next = false;       // the next launch goes directly behind this node's K/V append kernel

    int map_slot(const CUtensorMap &m) {
        for (int i = 0; i < n_maps; i++)
            if (!memcmp(&p.maps[i], &m, sizeof m)) return i;
        if (n_maps == QW_MAX_MAPS) return -1;
        p.maps[n_maps] = m;
        return n_maps++;
    }
    bool flush() {
        if (!n) return true;
        p.n_seq = n;
        p.early = early_next ? 1 : 0;
        early_next = false;
        const bool ok = run_split(c, p, max_rows);
        n = 0; n_maps = 0; max_rows = 0;
        return ok;
    }
    bool add(const AttnSeq &sq, const CUtensorMap &km, const CUtensorMap &vm) {
        for (int attempt = 0; attempt < 2; attempt++) {
            const int saved = n_maps;
            const int k = n < QW_MAX_SEQ ? map_slot(km) : -1;
            const int v = k >= 0 ? map_slot(vm) : -1;
            if (k >= 0 && v >= 0) {
                p.seq[n] = sq;
                p.seq[n].kmap = (uint8_t)k; p.seq[n].vmap = (uint8_t)v;
                max_rows = std::max(max_rows, sq.rows);
                n++;
                return true;
            }
            n_maps = saved;
            if (!flush()) return false;
        }
        return false;
    }
};

// The tcgen05 prefill kernel over one sequence: q_bf16 is [rows, q_heads, 256] in device memory.
// With cs_table != nullptr, q_bf16 is instead the raw [rows, q_heads, 512] bf16 [q|gate] input: the kernel
// norms (weights q_norm_w or nullptr, eps) and rotates its own query tiles, with the angles' cos / sin from
// cs_table ([rows, 64] f32, left by the pre-op).
bool run_prefill(qw_cmd c, const __nv_bfloat16 *q_bf16, void *out, int out_dtype, const void *gate, int gate_dtype,
                 int gate_stride, qw_ref kcache, qw_ref vcache, int32_t rows, int32_t q_heads, int32_t kv_heads,
                 int32_t max_ctx, int32_t base_pos, float scale, const float *cs_table = nullptr,
                 const uint16_t *q_norm_w = nullptr, float eps = 0.0f) {
    PrefillParams p;
    memset(&p, 0, sizeof p);
    int64_t k_rows = 0, v_rows = 0;
    if (!resolve_cache(c, kcache, kv_heads, max_ctx, QW_HEAD_DIM, base_pos + rows, false, false, &p.kc, &p.kmap, 64, &k_rows)) return false;
    if (!resolve_cache(c, vcache, kv_heads, max_ctx, QW_HEAD_DIM, base_pos + rows, false, false, &p.vc, &p.vmap, 64, &v_rows)) return false;
    p.q = q_bf16;
    p.out = out; p.out_dtype = out_dtype; p.gate = gate; p.gate_dtype = gate_dtype; p.gate_stride = gate_stride;
    p.rows = rows; p.base_pos = base_pos; p.q_heads = q_heads; p.kv_heads = kv_heads; p.gqa = q_heads / kv_heads;
    p.n_q_tiles = (rows + 127) / 128;
    p.oob_row = (int32_t)std::min<int64_t>(std::max(k_rows, v_rows), 0x7fffffff);
    p.scale = scale;
    p.status = cmd_status(c);
    const uint64_t row = (uint64_t)q_heads * 256;
    p.fuse_q = cs_table != nullptr; p.q_norm_w = q_norm_w; p.eps = eps;
    if (p.fuse_q && !encode_tile_map(&p.csmap, cs_table, DT_F32, 64, 64, rows)) return cmd_fail(c, "%s", "prefill: tensor map encoding failed"), false;
    if (!encode_tile_map(&p.qmap, q_bf16, DT_BF16, p.fuse_q ? 2 * row - 256 : row, p.fuse_q ? 2 * row : row, rows) ||
        !encode_tile_map(&p.omap, out, out_dtype, row, row, rows) ||
        (gate && !encode_tile_map(&p.gmap, gate, gate_dtype, (uint64_t)(q_heads - 1) * gate_stride + 256, (uint64_t)q_heads * gate_stride, rows)))
        return cmd_fail(c, "%s", "prefill: tensor map encoding failed"), false;
    KTime kt = {nullptr, nullptr, "qw_attn_prefill"};
    const bool timed = SH.time_kernels && cudaEventCreate(&kt.t0) == cudaSuccess && cudaEventCreate(&kt.t1) == cudaSuccess;
    if (timed) cudaEventRecord(kt.t0, c->stream);
    launch_attn_prefill(c->stream, p);
    if (timed) { cudaEventRecord(kt.t1, c->stream); c->ktimes.push_back(kt); }
    return cuda_ok(c, cudaGetLastError(), "prefill launch");
}

// An op may encode on c: the backend is up and c has not failed.  The command buffer's device
// becomes the current one (a host that drives several GPUs alternates between their command buffers).
bool live(qw_cmd c) {
    if (!c || c->failed || !g_devs[c->device].up) return false;
    use_device(c->device);
    return true;
}


}  // namespace

// ---------------------------------------------------------------------------------------
// lifecycle
// ---------------------------------------------------------------------------------------
// Brings up CUDA device `dev` (made current) as g_devs[dev].
static bool init_device(int dev, char *err, size_t errcap) {
    auto fail = [&](const char *fmt, const char *arg) {
        if (err && errcap) snprintf(err, errcap, fmt, arg);
        set_error(fmt, arg);
        return false;
    };
    if (dev < 0 || dev >= MAX_DEVICES) return fail("%s", "device index out of range");
    if (cudaSetDevice(dev) != cudaSuccess) return fail("%s", "cudaSetDevice failed");
    Globals &g = g_devs[dev];
    g_cur = &g;
    if (g.up) return true;
    g.device = dev;
    if (cudaGetDeviceProperties(&g.prop, dev) != cudaSuccess) return fail("%s", "cudaGetDeviceProperties failed");
    if (g.prop.major != 10) return fail("device %s is not compute capability 10.x (this backend is sm_100a only)", g.prop.name);
    snprintf(g.name, sizeof g.name, "%s", g.prop.name);
    g.sms = g.prop.multiProcessorCount > 0 ? g.prop.multiProcessorCount : 148;
    if (!entry("cuTensorMapEncodeTiled", &g.encodeTiled)) return fail("%s", "driver lacks cuTensorMapEncodeTiled");
    const bool vmm = entry("cuMemAddressReserve", &g.memAddressReserve) && entry("cuMemAddressFree", &g.memAddressFree) &&
                     entry("cuMemCreate", &g.memCreate) && entry("cuMemRelease", &g.memRelease) &&
                     entry("cuMemMap", &g.memMap) && entry("cuMemUnmap", &g.memUnmap) &&
                     entry("cuMemSetAccess", &g.memSetAccess) && entry("cuMemGetAllocationGranularity", &g.memGetGranularity);
    if (!vmm) g.memAddressReserve = nullptr;
    const size_t st_bytes = (size_t)STATUS_SLOTS * STATUS_STRIDE * sizeof(int);
    if (cudaHostAlloc((void **)&g.status_host, st_bytes, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void **)&g.status_dev, g.status_host, 0) != cudaSuccess)
        return fail("%s", "cannot allocate the status words");
    memset(g.status_host, 0, st_bytes);
    g.status_used = 1;
    if (cudaStreamCreateWithFlags(&g.copy_stream, cudaStreamNonBlocking) != cudaSuccess) g.copy_stream = nullptr;
    if (cudaStreamCreateWithFlags(&g.down_stream, cudaStreamNonBlocking) != cudaSuccess) g.down_stream = nullptr;
    g.up = true;
    return true;
}

extern "C" bool qw_gpu_init(char *err, size_t errcap) {
    if (G.up) return true;
    int n = 0, dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        const char *why = e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0";
        if (err && errcap) snprintf(err, errcap, "no CUDA device: %s", why);
        set_error("no CUDA device: %s", why);
        return false;
    }
    if (cudaGetDevice(&dev) != cudaSuccess) {
        if (err && errcap) snprintf(err, errcap, "cudaGetDevice failed");
        set_error("cudaGetDevice failed");
        return false;
    }
    if (!init_device(dev, err, errcap)) return false;
    SH.has_error = false;
    return true;
}

extern "C" int32_t qw_gpu_device_count(void) {
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess ? n : 0;
}

// Devices 0 .. n_dev-1 of this process, each able to read and write the others' memory (the
// exchange of partials stores straight into a peer's buffer).  Device 0 is current afterwards.
extern "C" bool qw_gpu_init_multi(int32_t n_dev, char *err, size_t errcap) {
    const int have = qw_gpu_device_count();
    if (n_dev <= 0 || n_dev > have || n_dev > MAX_DEVICES) {
        if (err && errcap) snprintf(err, errcap, "%d devices asked for, %d present (at most %d)", n_dev, have, MAX_DEVICES);
        set_error("%d devices asked for, %d present", n_dev, have);
        return false;
    }
    for (int d = 0; d < n_dev; d++)
        if (!init_device(d, err, errcap)) return false;
    for (int d = 0; d < n_dev; d++) {
        cudaSetDevice(d);
        for (int o = 0; o < n_dev; o++) {
            if (o == d) continue;
            int can = 0;
            cudaDeviceCanAccessPeer(&can, d, o);
            cudaError_t e = can ? cudaDeviceEnablePeerAccess(o, 0) : cudaErrorPeerAccessUnsupported;
            if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
            if (e != cudaSuccess) {
                if (err && errcap) snprintf(err, errcap, "device %d cannot reach device %d: %s", d, o, cudaGetErrorString(e));
                set_error("device %d cannot reach device %d: %s", d, o, cudaGetErrorString(e));
                cudaGetLastError();
                return false;
            }
        }
    }
    cudaSetDevice(0);
    g_cur = &g_devs[0];
    SH.has_error = false;
    return true;
}

extern "C" bool qw_gpu_select(int32_t dev) {
    if (dev < 0 || dev >= MAX_DEVICES || !g_devs[dev].up) { set_error("qw_gpu_select: device %d was not initialised", dev); return false; }
    use_device(dev);
    return true;
}
extern "C" int32_t qw_gpu_current(void) { return G.up ? G.device : -1; }

extern "C" void qw_gpu_shutdown(void) {
    for (int d = 0; d < MAX_DEVICES; d++) {
        Globals &g = g_devs[d];
        if (!g.up) continue;
        cudaSetDevice(d);
        cudaDeviceSynchronize();
        for (auto &s : g.scratch_pool) cudaFree(s.p);
        g.scratch_pool.clear();
        for (auto &st : g.stream_pool) cudaStreamDestroy(st);
        g.stream_pool.clear();
        if (g.copy_stream) { cudaStreamDestroy(g.copy_stream); g.copy_stream = nullptr; }
        if (g.down_stream) { cudaStreamDestroy(g.down_stream); g.down_stream = nullptr; }
        g.map_cache.clear();
        if (g.status_host) cudaFreeHost(g.status_host);
        g.status_host = g.status_dev = nullptr;
        g.up = false;
    }
}

extern "C" const char *qw_gpu_name(void) { return G.up ? G.name : "(no device)"; }
extern "C" uint64_t qw_gpu_working_set_limit(void) { return G.up ? (uint64_t)G.prop.totalGlobalMem : 0; }
extern "C" uint64_t qw_gpu_max_buffer_length(void) { return G.up ? (uint64_t)G.prop.totalGlobalMem : 0; }
extern "C" const char *qw_gpu_last_error(void) { return SH.has_error ? SH.last_error : nullptr; }
extern "C" int32_t qw_gpu_sm_count(void) { return G.up ? sm_count() : 0; }
extern "C" uint64_t qw_gpu_launch_count(void) { return (uint64_t)qw::g_launches; }
extern "C" bool qw_gpu_tune(const char *knob, int32_t value) {
    if (knob && !strcmp(knob, "split_kg") && (value == 4 || value == 6)) { qw::g_tune_split_kg = value; return true; }
    if (knob && !strcmp(knob, "prefill_tc") && (value == 0 || value == 1)) { qw::g_tune_prefill_tc = value; return true; }
    if (knob && !strcmp(knob, "prefill_fuse_q") && (value == 0 || value == 1)) { qw::g_tune_prefill_fuse_q = value; return true; }
    if (knob && !strcmp(knob, "pdl") && (value == 0 || value == 1)) { qw::g_tune_pdl = value; return true; }
    if (knob && !strcmp(knob, "masked_tc") && value >= 0 && value <= 2) { qw::g_tune_masked_tc = value; return true; }
    if (knob && !strcmp(knob, "split_kg2") && (value == 2 || value == 3)) { qw::g_tune_split_kg2 = value; return true; }
    if (knob && !strcmp(knob, "qmv_tc") && (value == 0 || value == 1)) { qw::g_tune_qmv_tc = value; return true; }
    if (knob && !strcmp(knob, "qmv_pre") && value >= 0 && value <= 2) { qw::g_tune_qmv_pre = value; return true; }
    if (knob && !strcmp(knob, "qmm_tc") && (value == 0 || value == 1)) { qw::g_tune_qmm_tc = value; return true; }
    return false;
}
// How the split-KV kernel would divide a launch: pure host arithmetic, no device needed.
extern "C" int32_t qw_attn_split_plan(int32_t n_seq, int32_t kv_heads, const int32_t *n_keys, int32_t n_cta_max,
                                      int32_t *share_first, int32_t *needs_merge) {
    if (n_seq <= 0 || n_seq > QW_MAX_SEQ || kv_heads <= 0 || !n_keys || n_cta_max <= 0 || !share_first) return 0;
    AttnParams p;
    memset(&p, 0, sizeof p);
    p.n_seq = n_seq; p.kv_heads = kv_heads;
    int cum = 0;
    for (int i = 0; i < n_seq; i++) {
        if (n_keys[i] <= 0) return 0;
        p.seq[i].key_lo = 0; p.seq[i].key_hi = n_keys[i];
        p.seq[i].tile0 = 0; p.seq[i].n_tiles = (n_keys[i] + 31) / 32; p.seq[i].cum_tiles = cum;
        cum += p.seq[i].n_tiles * kv_heads;
    }
    p.total_tiles = cum;
    p.n_cta = std::min(std::min(n_cta_max, 256), cum);
    attn_split_shares(p, share_first);
    if (needs_merge) *needs_merge = attn_split_needs_merge(p) ? 1 : 0;
    return p.n_cta;
}
extern "C" void qw_prof_kernels(bool on) { SH.time_kernels = on; }
extern "C" bool qw_prof_kernel_read(const char *kernel, double *ms_total, int64_t *launches, bool reset) {
    auto it = SH.kernel_ms.find(kernel ? kernel : "");
    if (it == SH.kernel_ms.end()) { if (ms_total) *ms_total = 0; if (launches) *launches = 0; return false; }
    if (ms_total) *ms_total = it->second.first;
    if (launches) *launches = it->second.second;
    if (reset) SH.kernel_ms.erase(it);
    return true;
}

// ---------------------------------------------------------------------------------------
// buffers
// ---------------------------------------------------------------------------------------
extern "C" qw_buf qw_buf_alloc(size_t len) {
    if (!G.up) { set_error("qw_buf_alloc before qw_gpu_init"); return nullptr; }
    qw_buf b = new qw_buf_s{BUF_SHARED, len, nullptr, nullptr, true, true, false, nullptr};
    b->device = G.device;
    const size_t n = std::max<size_t>(len, 16);
    if (cudaHostAlloc(&b->host, n, cudaHostAllocDefault) != cudaSuccess || cudaMalloc(&b->dev, n) != cudaSuccess) {
        set_error("cannot allocate a %zu-byte shared buffer", len);
        if (b->host) cudaFreeHost(b->host);
        delete b;
        cudaGetLastError();
        return nullptr;
    }
    memset(b->host, 0, n);
    cudaMemset(b->dev, 0, n);
    cudaStreamSynchronize(0);   // the fill must not trail kernels launched on other streams
    return b;
}

extern "C" qw_buf qw_buf_wrap(void *ptr, size_t len) {
    if (!G.up || !ptr) return nullptr;
    qw_buf b = new qw_buf_s{BUF_SHARED, len, ptr, nullptr, false, true, false, nullptr};
    b->device = G.device;
    if (cudaMalloc(&b->dev, std::max<size_t>(len, 16)) != cudaSuccess) { set_error("cannot mirror a %zu-byte wrapped buffer", len); delete b; cudaGetLastError(); return nullptr; }
    if (cudaHostRegister(ptr, len, cudaHostRegisterDefault) == cudaSuccess) b->registered = true;
    else cudaGetLastError();   // pageable memory still works, copies are just staged
    return b;
}

extern "C" qw_buf qw_buf_alloc_device(size_t len) {
    if (!G.up) { set_error("qw_buf_alloc_device before qw_gpu_init"); return nullptr; }
    qw_buf b = new qw_buf_s{BUF_DEVICE, len, nullptr, nullptr, false, true, false, nullptr};
    b->device = G.device;
    if (cudaMalloc(&b->dev, std::max<size_t>(len, 16)) != cudaSuccess) { set_error("cannot allocate %zu bytes of device memory", len); delete b; cudaGetLastError(); return nullptr; }
    cudaMemset(b->dev, 0, std::max<size_t>(len, 16));
    cudaStreamSynchronize(0);
    return b;
}

extern "C" qw_buf qw_buf_wrap_device(void *device_ptr, size_t len) {
    if (!G.up || !device_ptr) return nullptr;
    qw_buf b = new qw_buf_s{BUF_DEVICE, len, nullptr, device_ptr, false, false, false, nullptr};
    b->device = G.device;
    return b;
}

extern "C" void qw_buf_free(qw_buf b) {
    if (!b) return;
    if (b->kind == BUF_ARENA) { arena_destroy(b->arena); delete b; return; }
    if (b->kind == BUF_POOL) { pool_release(b->pool); delete b; return; }      // the memory goes with its last arena
    use_device(b->device);
    // work that still uses the buffer must finish first; tensor maps built over it are dropped
    if (b->own_dev || b->registered) cudaDeviceSynchronize();
    const uintptr_t lo = (uintptr_t)b->dev, hi = lo + b->len;
    for (auto it = G.map_cache.begin(); it != G.map_cache.end();)
        it = (it->first.first >= lo && it->first.first < hi) ? G.map_cache.erase(it) : std::next(it);
    if (b->registered) cudaHostUnregister(b->host);
    if (b->own_host && b->host) cudaFreeHost(b->host);
    if (b->own_dev && b->dev) cudaFree(b->dev);
    delete b;
}

extern "C" void *qw_buf_contents(qw_buf b) { return b && b->kind == BUF_SHARED ? b->host : nullptr; }
extern "C" size_t qw_buf_length(qw_buf b) { return b ? b->len : 0; }
extern "C" void *qw_buf_device_ptr(qw_buf b) { return b ? b->dev : nullptr; }

extern "C" bool qw_buf_upload(qw_buf b, size_t off, const void *src, size_t len) {
    if (!b || b->kind == BUF_ARENA || b->kind == BUF_POOL || off + len > b->len) { set_error("qw_buf_upload: bad range"); return false; }
    use_device(b->device);
    if (b->kind == BUF_SHARED) memcpy((char *)b->host + off, src, len);
    if (cudaMemcpy((char *)b->dev + off, src, len, cudaMemcpyHostToDevice) != cudaSuccess) { set_error("qw_buf_upload: copy failed"); return false; }
    return true;
}
extern "C" bool qw_buf_download(qw_buf b, size_t off, void *dst, size_t len) {
    if (!b || b->kind == BUF_ARENA || b->kind == BUF_POOL || off + len > b->len) { set_error("qw_buf_download: bad range"); return false; }
    use_device(b->device);
    if (cudaMemcpy(dst, (char *)b->dev + off, len, cudaMemcpyDeviceToHost) != cudaSuccess) { set_error("qw_buf_download: copy failed"); return false; }
    return true;
}

// ---------------------------------------------------------------------------------------
// arena API
// ---------------------------------------------------------------------------------------
static qw_buf arena_new(Pool *pool, bool private_pool, int32_t n_layers, int32_t kv_heads, int32_t max_ctx, int32_t head_dim,
                        uint32_t shuffle_seed) {
    if (n_layers <= 0 || kv_heads <= 0 || max_ctx <= 0 || head_dim != QW_HEAD_DIM) { set_error("arena: unsupported shape"); return nullptr; }
    Arena *a = new Arena();
    a->n_layers = n_layers; a->kv_heads = kv_heads; a->max_ctx = max_ctx; a->head_dim = head_dim;
    a->pages_per_head = (max_ctx + QW_PAGE_TOKENS - 1) / QW_PAGE_TOKENS;
    a->max_pages = (int64_t)n_layers * kv_heads * a->pages_per_head;
    a->in_use = 0; a->table_dev = nullptr;
    if (private_pool) {
        pool = pool_create((size_t)a->max_pages * PAGE_BYTES, shuffle_seed);
        if (!pool) { delete a; return nullptr; }
    } else {
        pool->refs++;
    }
    a->pool = pool;
    a->table_host.assign((size_t)a->max_pages, -1);
    if (cudaMalloc(&a->table_dev, (size_t)a->max_pages * sizeof(int32_t)) != cudaSuccess) { set_error("arena: cannot allocate the page table"); arena_destroy(a); cudaGetLastError(); return nullptr; }
    cudaMemset(a->table_dev, 0xff, (size_t)a->max_pages * sizeof(int32_t));
    cudaStreamSynchronize(0);   // the fill must not trail kernels launched on other streams
    qw_buf b = new qw_buf_s{BUF_ARENA, (size_t)n_layers * kv_heads * max_ctx * head_dim * 2, nullptr,
                            reinterpret_cast<void *>(pool->va), false, false, false, a};
    b->device = G.device;
    return b;
}
extern "C" qw_buf qw_kv_arena_alloc_ex(int32_t n_layers, int32_t kv_heads, int32_t max_ctx, int32_t head_dim,
                                       uint32_t shuffle_seed) {
    if (!G.up) { set_error("qw_kv_arena_alloc before qw_gpu_init"); return nullptr; }
    return arena_new(nullptr, true, n_layers, kv_heads, max_ctx, head_dim, shuffle_seed);
}
extern "C" qw_buf qw_kv_arena_alloc(int32_t n_layers, int32_t kv_heads, int32_t max_ctx, int32_t head_dim) {
    return qw_kv_arena_alloc_ex(n_layers, kv_heads, max_ctx, head_dim, 0);
}
extern "C" qw_buf qw_kv_pool_alloc(size_t max_bytes, uint32_t shuffle_seed) {
    if (!G.up) { set_error("qw_kv_pool_alloc before qw_gpu_init"); return nullptr; }
    if (!max_bytes) { set_error("qw_kv_pool_alloc: empty pool"); return nullptr; }
    Pool *pl = pool_create(max_bytes, shuffle_seed);
    if (!pl) return nullptr;
    qw_buf b = new qw_buf_s{BUF_POOL, pl->va_size, nullptr, reinterpret_cast<void *>(pl->va), false, false, false, nullptr};
    b->pool = pl;
    b->device = G.device;
    return b;
}
extern "C" qw_buf qw_kv_arena_alloc_in(qw_buf pool, int32_t n_layers, int32_t kv_heads, int32_t max_ctx, int32_t head_dim) {
    if (!pool || pool->kind != BUF_POOL) { set_error("qw_kv_arena_alloc_in: not a pool"); return nullptr; }
    use_device(pool->device);
    return arena_new(pool->pool, false, n_layers, kv_heads, max_ctx, head_dim, 0);
}
extern "C" int64_t qw_kv_pool_bytes_committed(qw_buf pool) {
    if (!pool || pool->kind != BUF_POOL) return -1;
    return pool->pool->vmm ? (int64_t)(pool->pool->chunks.size() * CHUNK_BYTES) : (int64_t)pool->pool->va_size;
}

static bool kv_rw(qw_buf cache, int32_t layer, int32_t head, int32_t pos0, int32_t n, void *host, bool store,
                  int32_t kv_heads, int32_t max_ctx, int32_t head_dim) {
    if (!cache || n < 0 || pos0 < 0 || head_dim != QW_HEAD_DIM || (int64_t)pos0 + n > max_ctx || head < 0 || head >= kv_heads) {
        set_error("qw_kv_read/store: bad arguments");
        return false;
    }
    const size_t row = (size_t)head_dim * 2;
    if (cache->kind == BUF_ARENA) {
        Arena *a = cache->arena;
        if (a->kv_heads != kv_heads || a->max_ctx != max_ctx || layer < 0 || layer >= a->n_layers) { set_error("qw_kv_read/store: shape differs from the arena's"); return false; }
        use_device(cache->device);
        if (store && !arena_ensure(a, layer, pos0, pos0 + n, 0)) return false;
        const int32_t *tab = a->table_host.data() + ((size_t)layer * a->kv_heads + head) * a->pages_per_head;
        int t = pos0;
        char *hp = (char *)host;
        while (t < pos0 + n) {
            const int pg = t / QW_PAGE_TOKENS, in = t % QW_PAGE_TOKENS;
            const int cnt = std::min(QW_PAGE_TOKENS - in, pos0 + n - t);
            if (tab[pg] < 0) {
                if (store) { set_error("qw_kv_store: page not mapped"); return false; }
                memset(hp, 0, (size_t)cnt * row);   // never written: reads as zeros
            } else {
                char *dp = (char *)a->pool->va + ((size_t)tab[pg] * QW_PAGE_TOKENS + in) * row;
                if (cudaMemcpy(store ? (void *)dp : (void *)hp, store ? (void *)hp : (void *)dp, (size_t)cnt * row,
                               store ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost) != cudaSuccess) {
                    set_error("qw_kv_read/store: copy failed");
                    return false;
                }
            }
            t += cnt;
            hp += (size_t)cnt * row;
        }
        return true;
    }
    const size_t off = (((size_t)layer * kv_heads + head) * max_ctx + pos0) * row;
    if (off + (size_t)n * row > cache->len) { set_error("qw_kv_read/store: range exceeds the buffer"); return false; }
    if (store) return qw_buf_upload(cache, off, host, (size_t)n * row);
    return qw_buf_download(cache, off, host, (size_t)n * row);
}
extern "C" bool qw_kv_read(qw_buf cache, int32_t layer, int32_t head, int32_t pos0, int32_t n, void *dst,
                           int32_t kv_heads, int32_t max_ctx, int32_t head_dim) {
    return kv_rw(cache, layer, head, pos0, n, dst, false, kv_heads, max_ctx, head_dim);
}
extern "C" bool qw_kv_store(qw_buf cache, int32_t layer, int32_t head, int32_t pos0, int32_t n, const void *src,
                            int32_t kv_heads, int32_t max_ctx, int32_t head_dim) {
    return kv_rw(cache, layer, head, pos0, n, const_cast<void *>(src), true, kv_heads, max_ctx, head_dim);
}

// The KV section of the reference's packed session state (qwasar_graph.c:296-303): layer by layer,
// head by head, the K rows of the first n_tokens positions then the V rows.  One gather (or scatter)
// kernel and one copy per layer through a staging buffer.
static bool kv_pack_io(qw_buf kcache, qw_buf vcache, int32_t n_layers, int32_t kv_heads, int32_t max_ctx, int32_t head_dim,
                       int32_t n_tokens, void *host, size_t len, bool unpack) {
    if (kcache) use_device(kcache->device);
    if (!G.up || !kcache || !vcache || n_layers <= 0 || kv_heads <= 0 || head_dim != QW_HEAD_DIM || n_tokens < 0 || n_tokens > max_ctx || !host) {
        set_error("qw_kv_pack/unpack: bad arguments");
        return false;
    }
    const size_t layer_packed = (size_t)kv_heads * 2 * n_tokens * head_dim * 2;
    if (len != layer_packed * n_layers) { set_error("qw_kv_pack/unpack: %zu bytes given, the state is %zu", len, layer_packed * n_layers); return false; }
    if (n_tokens == 0) return true;
    qw_cmd c = qw_cmd_begin();
    if (!c) return false;
    void *stage = cmd_scratch(c, layer_packed);
    const size_t layer_bytes = (size_t)kv_heads * max_ctx * head_dim * 2;
    bool ok = stage != nullptr;
    for (int32_t l = 0; ok && l < n_layers; l++) {
        KvLayer kc, vc;
        ok = resolve_cache(c, qw_ref{kcache, l * layer_bytes}, kv_heads, max_ctx, head_dim, n_tokens, unpack, unpack, &kc, nullptr) &&
             resolve_cache(c, qw_ref{vcache, l * layer_bytes}, kv_heads, max_ctx, head_dim, n_tokens, unpack, unpack, &vc, nullptr);
        if (!ok) break;
        char *hp = (char *)host + (size_t)l * layer_packed;
        if (unpack) ok = cuda_ok(c, cudaMemcpyAsync(stage, hp, layer_packed, cudaMemcpyHostToDevice, c->stream), "unpack copy");
        if (ok) launch_kv_pack(c->stream, kc, vc, stage, kv_heads, n_tokens, unpack);
        if (ok && !unpack) ok = cuda_ok(c, cudaMemcpyAsync(hp, stage, layer_packed, cudaMemcpyDeviceToHost, c->stream), "pack copy");
        // the staging buffer is reused by the next layer: the copy of this one must have left it
        if (ok) ok = cuda_ok(c, cudaStreamSynchronize(c->stream), "pack");
    }
    qw_cmd_wait(c);
    if (c->failed) { set_error("%s", c->err); ok = false; }
    qw_cmd_free(c);
    return ok;
}
extern "C" size_t qw_kv_state_bytes(int32_t n_layers, int32_t kv_heads, int32_t head_dim, int32_t n_tokens) {
    if (n_layers <= 0 || kv_heads <= 0 || head_dim <= 0 || n_tokens <= 0) return 0;
    return (size_t)n_layers * kv_heads * 2 * n_tokens * head_dim * 2;
}
extern "C" uint32_t qw_kv_element_tag(void) { return 0x36314642u; }     // "BF16"
extern "C" bool qw_kv_pack(qw_buf kcache, qw_buf vcache, int32_t n_layers, int32_t kv_heads, int32_t max_ctx, int32_t head_dim,
                           int32_t n_tokens, void *dst, size_t cap) {
    const size_t need = qw_kv_state_bytes(n_layers, kv_heads, head_dim, n_tokens);
    if (cap < need) { set_error("qw_kv_pack: %zu bytes given, the state is %zu", cap, need); return false; }
    return kv_pack_io(kcache, vcache, n_layers, kv_heads, max_ctx, head_dim, n_tokens, dst, need, false);
}
extern "C" bool qw_kv_unpack(qw_buf kcache, qw_buf vcache, int32_t n_layers, int32_t kv_heads, int32_t max_ctx, int32_t head_dim,
                             int32_t n_tokens, const void *src, size_t len) {
    return kv_pack_io(kcache, vcache, n_layers, kv_heads, max_ctx, head_dim, n_tokens, const_cast<void *>(src), len, true);
}

extern "C" void qw_kv_arena_trim(qw_buf cache, int32_t n_tokens) {
    if (!cache || cache->kind != BUF_ARENA) return;
    Arena *a = cache->arena;
    use_device(cache->device);
    cudaDeviceSynchronize();
    const int keep = (std::max(n_tokens, 0) + QW_PAGE_TOKENS - 1) / QW_PAGE_TOKENS;
    for (size_t lh = 0; lh < (size_t)a->n_layers * a->kv_heads; lh++) {
        int32_t *row = a->table_host.data() + lh * a->pages_per_head;
        bool any = false;
        for (int pg = keep; pg < a->pages_per_head; pg++)
            if (row[pg] >= 0) { a->pool->free_pages.push_back(row[pg]); row[pg] = -1; a->in_use--; any = true; }
        if (any && keep < a->pages_per_head)
            cudaMemcpy(a->table_dev + lh * a->pages_per_head + keep, row + keep, (size_t)(a->pages_per_head - keep) * sizeof(int32_t),
                       cudaMemcpyHostToDevice);
    }
}
extern "C" int64_t qw_kv_arena_pages_in_use(qw_buf cache) { return cache && cache->kind == BUF_ARENA ? cache->arena->in_use : -1; }
extern "C" int64_t qw_kv_arena_bytes_committed(qw_buf cache) {
    if (!cache || cache->kind != BUF_ARENA) return -1;
    Pool *pl = cache->arena->pool;
    return pl->vmm ? (int64_t)(pl->chunks.size() * CHUNK_BYTES) : (int64_t)pl->va_size;
}

// ---------------------------------------------------------------------------------------
// command buffers
// ---------------------------------------------------------------------------------------
static qw_cmd cmd_new(cudaStream_t s, bool own) {
    qw_cmd c = new qw_cmd_s();
    c->stream = s; c->own_stream = own; c->failed = false; c->err[0] = 0; c->parallel = 0;
    c->device = G.device;
    // a status word of its own, so that a kernel's bounded wait that ran out is reported on the
    // command buffer that launched it; with every slot taken the shared word 0 serves
    c->status_slot = 0;
    for (int i = 1; i < STATUS_SLOTS; i++)
        if (!(G.status_used >> i & 1)) { G.status_used |= (uint64_t)1 << i; c->status_slot = i; G.status_host[i * STATUS_STRIDE] = 0; break; }
    return c;
}
extern "C" qw_cmd qw_cmd_begin(void) {
    if (!G.up) return nullptr;
    cudaStream_t s;
    if (!G.stream_pool.empty()) {
        s = G.stream_pool.back();
        G.stream_pool.pop_back();
    } else if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) {
        set_error("cannot create a stream");
        return nullptr;
    }
    qw_cmd c = cmd_new(s, true);
    if (qw_prof_enabled()) qw_cmd_mark(c, nullptr);
    return c;
}
extern "C" qw_cmd qw_cmd_begin_on_stream(void *cuda_stream) {
    if (!G.up) return nullptr;
    return cmd_new(reinterpret_cast<cudaStream_t>(cuda_stream), false);
}
extern "C" void qw_cmd_commit(qw_cmd c) { if (c) cudaStreamQuery(c->stream); }
// qw_cmd_flush: "what is encoded so far may start" (qwasar_gpu.h:60-64; the reference's forward flushes every few
// layers, qwasar_flash_graph.c:657).  Ops launch as they are encoded here, so
// the hint is used for the other direction: the shared ranges written so far start their way back to the host on a
// stream of their own, behind an event on the command's stream, and qw_cmd_wait finds them done -- the outputs of
// a layer travel while the next layers run.  (A range written again later is simply copied again at the wait.)
extern "C" void qw_cmd_flush(qw_cmd c) {
    if (!c) return;
    use_device(c->device);
    bool any = false;
    for (auto &t : c->touched) any |= t.whi > t.wlo;
    if (!any || !G.down_stream) { cudaStreamQuery(c->stream); return; }
    if (!c->written && cudaEventCreateWithFlags(&c->written, cudaEventDisableTiming) != cudaSuccess) { c->written = nullptr; return; }
    if (!c->downloaded && cudaEventCreateWithFlags(&c->downloaded, cudaEventDisableTiming) != cudaSuccess) { c->downloaded = nullptr; return; }
    if (!cuda_ok(c, cudaEventRecord(c->written, c->stream), "flush event") ||
        !cuda_ok(c, cudaStreamWaitEvent(G.down_stream, c->written, 0), "flush wait")) return;
    for (auto &t : c->touched)
        if (t.whi > t.wlo) {
            cuda_ok(c, cudaMemcpyAsync((char *)t.b->host + t.wlo, (char *)t.b->dev + t.wlo, t.whi - t.wlo, cudaMemcpyDeviceToHost, G.down_stream), "download");
            t.wlo = t.whi = 0;
        }
    cuda_ok(c, cudaEventRecord(c->downloaded, G.down_stream), "download event");
    c->early_down = true;
}
extern "C" void qw_cmd_parallel(qw_cmd c, bool on) { if (c) c->parallel += on ? 1 : (c->parallel > 0 ? -1 : 0); }

extern "C" void qw_cmd_wait(qw_cmd c) {
    if (!c) return;
    use_device(c->device);
    for (auto &t : c->touched)
        if (t.whi > t.wlo)
            cuda_ok(c, cudaMemcpyAsync((char *)t.b->host + t.wlo, (char *)t.b->dev + t.wlo, t.whi - t.wlo, cudaMemcpyDeviceToHost, c->stream), "download");
    c->touched.clear();
    cudaError_t e = cudaStreamSynchronize(c->stream);
    if (e == cudaSuccess && c->early_down) { e = cudaEventSynchronize(c->downloaded); c->early_down = false; }
    if (e != cudaSuccess) cmd_fail(c, "GPU fault: %s", cudaGetErrorString(e));
    if (G.status_host) {
        volatile int *st = G.status_host + (size_t)c->status_slot * STATUS_STRIDE;
        if (*st != 0) {
            cmd_fail(c, "%s", status_text(*st));
            *st = 0;
        }
    }
    if (c->marks.size() > 1) {
        for (size_t i = 1; i < c->marks.size(); i++) {
            float ms = 0;
            if (c->marks[i].label && cudaEventElapsedTime(&ms, c->marks[i - 1].ev, c->marks[i].ev) == cudaSuccess) {
                auto &slot = SH.prof_ms[c->marks[i].label];
                slot.first += ms; slot.second++;
            }
        }
    }
    for (auto &m : c->marks) cudaEventDestroy(m.ev);
    c->marks.clear();
    for (auto &k : c->ktimes) {
        float ms = 0;
        if (cudaEventElapsedTime(&ms, k.t0, k.t1) == cudaSuccess) {
            auto &slot = SH.kernel_ms[k.kernel];
            slot.first += ms; slot.second++;
        }
        cudaEventDestroy(k.t0); cudaEventDestroy(k.t1);
    }
    c->ktimes.clear();
}

extern "C" void qw_cmd_free(qw_cmd c) {
    if (!c) return;
    use_device(c->device);
    if (c->status_slot) G.status_used &= ~((uint64_t)1 << c->status_slot);
    if (!c->touched.empty() || !c->scratch.empty()) cudaStreamSynchronize(c->stream);
    for (auto &s : c->scratch) G.scratch_pool.push_back(s);
    if (c->uploaded) cudaEventDestroy(c->uploaded);
    if (c->written) cudaEventDestroy(c->written);
    if (c->downloaded) cudaEventDestroy(c->downloaded);
    for (auto &m : c->marks) cudaEventDestroy(m.ev);
    for (auto &k : c->ktimes) { cudaEventDestroy(k.t0); cudaEventDestroy(k.t1); }
    if (c->own_stream) {
        // everything on the stream has been waited for (or is synchronised here) before reuse
        if (cudaStreamQuery(c->stream) != cudaSuccess) cudaStreamSynchronize(c->stream);
        if (c->failed || G.stream_pool.size() >= 16) cudaStreamDestroy(c->stream);
        else G.stream_pool.push_back(c->stream);
    }
    delete c;
}
extern "C" const char *qw_cmd_error(qw_cmd c) { return c && c->failed ? c->err : nullptr; }

extern "C" bool qw_prof_enabled(void) {
    if (SH.prof < 0) { const char *v = getenv("QWASAR_PROFILE"); SH.prof = (v && *v && strcmp(v, "0")) ? 1 : 0; }
    return SH.prof == 1;
}
extern "C" void qw_cmd_mark(qw_cmd c, const char *label) {
    if (!c || !qw_prof_enabled()) return;
    Mark m; m.label = label;
    if (cudaEventCreate(&m.ev) != cudaSuccess) return;
    cudaEventRecord(m.ev, c->stream);
    c->marks.push_back(m);
}
// The table of qwasar_metal.m:435-447: one line per label, milliseconds per token when a token
// count is given, the share of the total, the marks counted, then the total.
extern "C" void qw_prof_report(FILE *out, long tokens) {
    if (!out || SH.prof_ms.empty()) return;
    double total = 0;
    for (auto &kv : SH.prof_ms) total += kv.second.first;
    const double per = tokens > 0 ? (double)tokens : 1.0;
    fprintf(out, "GPU time by section%s:\n", tokens > 0 ? ", per decoded token" : "");
    for (auto &kv : SH.prof_ms)
        fprintf(out, "  %-22s %8.3f ms  %5.1f%%  (%ld marks)\n", kv.first.c_str(), kv.second.first / per,
                100.0 * kv.second.first / (total > 0 ? total : 1.0), kv.second.second);
    fprintf(out, "  %-22s %8.3f ms\n", "total", total / per);
}
extern "C" void qw_prof_reset(void) { SH.prof_ms.clear(); }

extern "C" void qw_op_copy(qw_cmd c, qw_ref dst, qw_ref src, size_t n) {
    if (!live(c) || !n) return;
    // Both sides are taken on the device: an earlier op of this command buffer may have written the
    // source, and then only its device mirror is current until qw_cmd_wait.  A shared destination
    // is copied back at wait like any op output.
    void *d = dev_range(c, dst, n, true, 1);
    const void *s = dev_range(c, src, n, false, 1);
    if (!d || !s) return;
    cuda_ok(c, cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToDevice, c->stream), "copy");
}

// ---------------------------------------------------------------------------------------
// pre/post ops (reference signatures)
// ---------------------------------------------------------------------------------------
extern "C" void qw_op_split_heads2(qw_cmd c, qw_ref a, qw_ref b, qw_ref src, int32_t rows, int32_t heads, int32_t dim) {
    if (!live(c) || rows <= 0 || heads <= 0 || dim <= 0) return;
    const size_t n = (size_t)rows * heads * dim * 4;
    float *pa = (float *)dev_range(c, a, n, true), *pb = (float *)dev_range(c, b, n, true);
    const float *ps = (const float *)dev_range(c, src, 2 * n, false);
    if (!pa || !pb || !ps) return;
    launch_split_heads2(c->stream, pa, pb, ps, rows, heads, dim);
}

extern "C" void qw_op_rms_norm(qw_cmd c, qw_ref y, qw_ref x, qw_ref weight, int32_t dim, int32_t rows, float eps, float out_scale) {
    if (!live(c) || rows <= 0 || dim <= 0) return;
    const size_t n = (size_t)rows * dim * 4;
    const float *px = (const float *)dev_range(c, x, n, false);
    float *py = (float *)dev_range(c, y, n, true);
    const uint16_t *pw = weight.buf ? (const uint16_t *)dev_range(c, weight, (size_t)dim * 2, false) : nullptr;
    if (!px || !py || (weight.buf && !pw)) return;
    launch_rms_norm(c->stream, py, px, pw, dim, rows, eps, out_scale);
}

extern "C" void qw_op_rope_partial(qw_cmd c, qw_ref x, qw_ref pos, qw_ref axis, qw_ref inv_freq, int32_t rows, int32_t heads,
                                   int32_t head_dim, int32_t rotary_dim) {
    if (!live(c) || rows <= 0 || heads <= 0 || rotary_dim <= 0 || rotary_dim > head_dim || (rotary_dim & 1)) return;
    float *px = (float *)dev_range(c, x, (size_t)rows * heads * head_dim * 4, true);
    const int32_t *pp = (const int32_t *)dev_range(c, pos, (size_t)3 * rows * 4, false, 4);
    const uint8_t *pa = (const uint8_t *)dev_range(c, axis, (size_t)rotary_dim / 2, false, 1);
    const float *pf = (const float *)dev_range(c, inv_freq, (size_t)rotary_dim / 2 * 4, false, 4);
    if (!px || !pp || !pa || !pf) return;
    launch_rope_partial(c->stream, px, pp, pa, pf, rows, heads, head_dim, rotary_dim);
}

extern "C" void qw_rope_tables(uint8_t *axis, float *inv_freq, int32_t rotary_dim, float theta, const int32_t mrope_section[3]) {
    // host arithmetic of qwasar_cpu.c:284-302: time axis by default, axes 1 and 2 on every
    // third frequency from their own offset, below three times their section
    const int32_t half = rotary_dim / 2;
    for (int32_t j = 0; j < half; j++) {
        uint8_t a = 0;
        if (j % 3 == 1 && j < std::min(mrope_section[1] * 3, half)) a = 1;
        if (j % 3 == 2 && j < std::min(mrope_section[2] * 3, half)) a = 2;
        axis[j] = a;
        inv_freq[j] = 1.0f / powf(theta, (float)(2 * j) / (float)rotary_dim);
    }
}

extern "C" void qw_op_mul_sigmoid(qw_cmd c, qw_ref y, qw_ref gate, int32_t n) {
    if (!live(c) || n <= 0) return;
    float *py = (float *)dev_range(c, y, (size_t)n * 4, true);
    const float *pg = (const float *)dev_range(c, gate, (size_t)n * 4, false);
    if (!py || !pg) return;
    launch_mul_sigmoid(c->stream, py, pg, n);
}

extern "C" void qw_op_slice_rows(qw_cmd c, qw_ref dst, qw_ref src, int32_t rows, int32_t src_stride, int32_t offset, int32_t len) {
    if (!live(c) || rows <= 0 || len <= 0) return;
    if (offset < 0 || offset + len > src_stride) { cmd_fail(c, "slice_rows: columns [%d, %d) outside rows of %d", offset, offset + len, src_stride); return; }
    float *pd = (float *)dev_range(c, dst, (size_t)rows * len * 4, true, 4);
    const float *ps = (const float *)dev_range(c, src, ((size_t)(rows - 1) * src_stride + offset + len) * 4, false, 4);
    if (!pd || !ps) return;
    launch_slice_rows(c->stream, pd, ps, rows, src_stride, offset, len);
}

extern "C" void qw_op_kv_write(qw_cmd c, qw_ref kcache, qw_ref vcache, qw_ref k, qw_ref v, int32_t rows, int32_t kv_heads,
                               int32_t head_dim, int32_t max_ctx, int32_t base_pos) {
    if (!live(c) || rows <= 0) return;
    if (head_dim != QW_HEAD_DIM) { fprintf(stderr, "qwasar: kv_write head_dim %d unsupported (kernel is built for 256)\n", head_dim); return; }
    if (kv_heads <= 0 || base_pos < 0 || (int64_t)base_pos + rows > max_ctx) { cmd_fail(c, "kv_write: positions [%d, %d) outside the cache", base_pos, base_pos + rows); return; }
    KvLayer kc, vc;
    if (!resolve_cache(c, kcache, kv_heads, max_ctx, head_dim, base_pos + rows, true, true, &kc, nullptr, 32, nullptr, base_pos)) return;
    if (!resolve_cache(c, vcache, kv_heads, max_ctx, head_dim, base_pos + rows, true, true, &vc, nullptr, 32, nullptr, base_pos)) return;
    const size_t n = (size_t)rows * kv_heads * head_dim * 4;
    const float *pk = (const float *)dev_range(c, k, n, false), *pv = (const float *)dev_range(c, v, n, false);
    if (!pk || !pv) return;
    launch_kv_write(c->stream, kc, vc, pk, pv, rows, kv_heads, base_pos);
}

// ---------------------------------------------------------------------------------------
// attention (reference signatures)
// ---------------------------------------------------------------------------------------
namespace {

struct AttnArgs {
    qw_ref out, q, gate, kcache, vcache;
    int32_t rows, base_pos;
};

// Rows of one call cut into chunks of at most 64 / gqa rows, each chunk a "sequence" of a
// split-KV launch.
bool attn_rows_split(qw_cmd c, const AttnArgs *seqs, int n_seq, int32_t q_heads, int32_t kv_heads, int32_t max_ctx,
                     float scale, int q_dtype, int out_dtype, int gate_dtype, int gate_stride) {
    const int gqa = q_heads / kv_heads;
    if (gqa > 64) return false;
    const int chunk_rows = std::max(1, 64 / gqa);
    const size_t q_el = q_dtype == DT_BF16 ? 2 : 4, o_el = out_dtype == DT_BF16 ? 2 : 4, g_el = gate_dtype == DT_BF16 ? 2 : 4;
    SplitBatch b;
    b.c = c;
    AttnParams &p = b.p;
    memset(&p, 0, sizeof p);
    p.q_heads = q_heads; p.kv_heads = kv_heads; p.gqa = gqa; p.q_dtype = q_dtype; p.out_dtype = out_dtype;
    p.gate_dtype = gate_dtype; p.gate_stride = gate_stride; p.scale = scale; p.mode = 0;
    for (int s = 0; s < n_seq; s++) {
        const AttnArgs &a = seqs[s];
        KvLayer kc, vc;
        CUtensorMap km, vm;
        if (!resolve_cache(c, a.kcache, kv_heads, max_ctx, QW_HEAD_DIM, a.base_pos + a.rows, false, false, &kc, &km)) return false;
        if (!resolve_cache(c, a.vcache, kv_heads, max_ctx, QW_HEAD_DIM, a.base_pos + a.rows, false, false, &vc, &vm)) return false;
        const size_t q_bytes = (size_t)a.rows * q_heads * 256 * q_el, o_bytes = (size_t)a.rows * q_heads * 256 * o_el;
        const char *qp = (const char *)dev_range(c, a.q, q_bytes, false);
        char *op = (char *)dev_range(c, a.out, o_bytes, true);
        const char *gp = a.gate.buf ? (const char *)dev_range(c, a.gate, ((size_t)a.rows * q_heads - 1) * gate_stride * g_el + 256 * g_el, false) : nullptr;
        if (!qp || !op || (a.gate.buf && !gp)) return false;
        for (int r0 = 0; r0 < a.rows; r0 += chunk_rows) {
            AttnSeq sq;
            memset(&sq, 0, sizeof sq);
            const int rr = std::min(chunk_rows, a.rows - r0);
            sq.q = qp + (size_t)r0 * q_heads * 256 * q_el;
            sq.out = op + (size_t)r0 * q_heads * 256 * o_el;
            sq.gate = gp ? gp + (size_t)r0 * q_heads * gate_stride * g_el : nullptr;
            sq.kc = kc; sq.vc = vc;
            sq.rows = rr; sq.base_pos = a.base_pos + r0;
            sq.key_lo = 0; sq.key_hi = a.base_pos + r0 + rr;
            if (!b.add(sq, km, vm)) return false;
        }
    }
    return b.flush();
}

}  // namespace

extern "C" void qw_op_attn_decode(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache, int32_t rows, int32_t q_heads,
                                  int32_t kv_heads, int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale) {
    if (!live(c)) return;
    if (head_dim != QW_HEAD_DIM) { fprintf(stderr, "qwasar: attention head_dim %d unsupported (kernel is built for 256)\n", head_dim); return; }
    if (!shape_ok(rows, q_heads, kv_heads, head_dim, max_ctx, base_pos)) { cmd_fail(c, "attn_decode: bad shape"); return; }
    AttnSeq sq;
    memset(&sq, 0, sizeof sq);
    if (!resolve_cache(c, kcache, kv_heads, max_ctx, head_dim, base_pos + rows, false, false, &sq.kc, nullptr)) return;
    if (!resolve_cache(c, vcache, kv_heads, max_ctx, head_dim, base_pos + rows, false, false, &sq.vc, nullptr)) return;
    const size_t n = (size_t)rows * q_heads * head_dim * 4;
    sq.q = dev_range(c, q, n, false);
    void *po = dev_range(c, out, n, true);
    if (!sq.q || !po) return;
    sq.rows = rows; sq.base_pos = base_pos; sq.key_lo = 0; sq.key_hi = base_pos + rows;
    const int splits = attn_per_query_splits(rows, q_heads, base_pos + rows);
    float *scr = (float *)cmd_scratch(c, attn_per_query_scratch_bytes(rows, q_heads, splits));
    if (!scr) return;
    float *pstat = scr + (size_t)splits * rows * q_heads * 256;
    launch_attn_per_query(c->stream, sq, q_heads, kv_heads, scale, scr, pstat, splits);
    launch_merge_parts(c->stream, po, DT_F32, scr, pstat, nullptr, DT_F32, 256, rows * q_heads, splits, nullptr, nullptr);
    cuda_ok(c, cudaGetLastError(), "attn_decode launch");
}

// ---- the 4-bit affine product (qwasar_gpu.h:84-118): one kernel behind all three names ----
static bool qmat_q4(qw_cmd c, const char *op, qw_ref y, qw_ref x, qw_ref w, qw_ref scales, qw_ref biases, int32_t k, int32_t n,
                    int32_t rows, int32_t group) {
    if (k <= 0 || n <= 0 || rows <= 0 || (group != 32 && group != 64) || k % group) {
        cmd_fail(c, "%s: k %d, n %d, rows %d, group %d (32 or 64, dividing k) not supported", op, k, n, rows, group);
        return false;
    }
    float *py = (float *)dev_range(c, y, (size_t)rows * n * 4, true, 4);
    const float *px = (const float *)dev_range(c, x, (size_t)rows * k * 4, false, 16);
    const uint32_t *pw = (const uint32_t *)dev_range(c, w, (size_t)n * (k / 8) * 4, false, 4);
    const uint16_t *ps = (const uint16_t *)dev_range(c, scales, (size_t)n * (k / group) * 2, false, 2);
    const uint16_t *pb = (const uint16_t *)dev_range(c, biases, (size_t)n * (k / group) * 2, false, 2);
    if (!py || !px || !pw || !ps || !pb) return false;
    // many tokens: the tcgen05 GEMM with the weights dequantised to fp16 in shared memory (fp16 operands, fp32
    // accumulation: the reference's tensor form and its bound, tests/test_qmv.c:117-131 -- a bound met from k = 2048
    // up, the shapes the reference tests it on: the rounding of the operands averages out with the square root of k)
    if (rows >= 16 && group == 64 && (k & 511) == 0 && k >= 2048 && (n & 7) == 0 && g_tune_qmm_tc &&
        ((reinterpret_cast<uintptr_t>(py) | reinterpret_cast<uintptr_t>(pw) | reinterpret_cast<uintptr_t>(ps) | reinterpret_cast<uintptr_t>(pb)) & 15) == 0) {
        void *x16 = cmd_scratch(c, qgemm_scratch_bytes(rows, k));
        QgemmParams gp;
        if (x16 && encode_2d_map(&gp.map_x, x16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)k, (uint64_t)k * 2, (uint64_t)rows, 64, 128, true) &&
            encode_2d_map(&gp.map_w, pw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)k / 8, (uint64_t)k / 2, (uint64_t)n, 8, 256, false) &&
            encode_2d_map(&gp.map_s, ps, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (uint64_t)k / 64, (uint64_t)k / 32, (uint64_t)n, 8, 256, false) &&
            encode_2d_map(&gp.map_b, pb, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (uint64_t)k / 64, (uint64_t)k / 32, (uint64_t)n, 8, 256, false)) {
            gp.y = py; gp.status = cmd_status(c); gp.rows = rows; gp.n = n; gp.k = k;
            if (launch_qgemm_q4(c->stream, gp, px, x16)) return cuda_ok(c, cudaGetLastError(), "qgemm_q4 launch");
            cudaGetLastError();
        }
    }
    const size_t xq_bytes = qmv_scratch_bytes(rows, k, group);
    launch_qmat_q4(c->stream, py, px, pw, ps, pb, k, n, rows, group, cmd_status(c), xq_bytes ? cmd_scratch(c, xq_bytes) : nullptr);
    return cuda_ok(c, cudaGetLastError(), "qmat_q4 launch");
}
extern "C" void qw_op_qmat_q4(qw_cmd c, qw_ref y, qw_ref x, qw_ref w, qw_ref scales, qw_ref biases, int32_t k, int32_t n, int32_t rows,
                              int32_t group) {
    if (live(c)) qmat_q4(c, "qmat_q4", y, x, w, scales, biases, k, n, rows, group);
}
extern "C" void qw_op_qmv_q4(qw_cmd c, qw_ref y, qw_ref x, qw_ref w, qw_ref scales, qw_ref biases, int32_t k, int32_t n, int32_t rows,
                             int32_t group) {
    if (live(c)) qmat_q4(c, "qmv_q4", y, x, w, scales, biases, k, n, rows, group);
}
extern "C" void qw_op_qmm_q4(qw_cmd c, qw_ref y, qw_ref x, qw_ref w, qw_ref scales, qw_ref biases, int32_t k, int32_t n, int32_t rows,
                             int32_t group) {
    if (live(c)) qmat_q4(c, "qmm_q4", y, x, w, scales, biases, k, n, rows, group);
}
extern "C" bool qw_op_qmv_q4_multi(qw_cmd c, qw_ref x, int32_t k, int32_t group, int32_t count, const qw_qmv_part *parts) {
    if (!live(c) || !parts || count <= 0 || count > 4 || k < 2048) return false;        // the reference's limits (qwasar_gpu.h:105-109)
    if ((group != 32 && group != 64) || k % group) { cmd_fail(c, "qmv_q4_multi: k %d, group %d not supported", k, group); return false; }
    QmvMulti m;
    memset(&m, 0, sizeof m);
    m.count = count; m.k = k; m.group = group;
    m.x = (const float *)dev_range(c, x, (size_t)k * 4, false, 16);
    if (!m.x) return false;
    bool aligned = true;
    for (int32_t i = 0; i < count; i++) {
        const int32_t n = parts[i].n;
        if (n <= 0) { cmd_fail(c, "qmv_q4_multi: part %d has no rows", i); return false; }
        m.n[i] = n;
        m.y[i] = (float *)dev_range(c, parts[i].y, (size_t)n * 4, true, 4);
        m.w[i] = (const uint32_t *)dev_range(c, parts[i].w, (size_t)n * (k / 8) * 4, false, 4);
        m.scales[i] = (const uint16_t *)dev_range(c, parts[i].scales, (size_t)n * (k / group) * 2, false, 2);
        m.biases[i] = (const uint16_t *)dev_range(c, parts[i].biases, (size_t)n * (k / group) * 2, false, 2);
        if (!m.y[i] || !m.w[i] || !m.scales[i] || !m.biases[i]) return false;
        aligned = aligned && ((uintptr_t)m.w[i] & 15) == 0;
    }
    if (aligned) {
        const size_t xq_bytes = qmv_scratch_bytes(1, k, group);
        launch_qmv_q4_multi(c->stream, m, cmd_status(c), xq_bytes ? cmd_scratch(c, xq_bytes) : nullptr);   // one dispatch for all parts
    } else {
        for (int32_t i = 0; i < count; i++) launch_qmat_q4(c->stream, m.y[i], m.x, m.w[i], m.scales[i], m.biases[i], k, m.n[i], 1, group, cmd_status(c), nullptr);
    }
    return cuda_ok(c, cudaGetLastError(), "qmv_q4_multi launch");
}

// ---- QSA indexer: block keys, block scores, selection (qwasar_gpu.h:620-639) ----
static bool qsa_shape_ok(qw_cmd c, const char *op, int32_t d, int32_t ratio, int32_t rotary_dim) {
    if (d <= 0 || d > 256 || d % 32 || ratio <= 0 || rotary_dim != 64 || d < 64) {
        cmd_fail(c, "%s: index head dim %d (a multiple of 32 up to 256), ratio %d, rotary_dim %d (64) not supported", op, d, ratio, rotary_dim);
        return false;
    }
    return true;
}
extern "C" void qw_op_qsa_pool(qw_cmd c, qw_ref pool, qw_ref ikeys, qw_ref k_norm, qw_ref inv_freq, int32_t d, int32_t ratio,
                               int32_t b0, int32_t b1, int32_t rotary_dim, float eps) {
    if (!live(c) || !qsa_shape_ok(c, "qsa_pool", d, ratio, rotary_dim)) return;
    if (b0 < 0 || b1 < b0) { cmd_fail(c, "qsa_pool: bad block range"); return; }
    if (b1 == b0) return;
    float *pp = (float *)dev_range(c, pool, (size_t)b1 * d * 4, true, 4);
    const float *pk = (const float *)dev_range(c, ikeys, (size_t)b1 * ratio * d * 4, false, 4);
    const uint16_t *pw = k_norm.buf ? (const uint16_t *)dev_range(c, k_norm, (size_t)d * 2, false, 2) : nullptr;
    const float *pf = (const float *)dev_range(c, inv_freq, 32 * 4, false, 4);
    if (!pp || !pk || !pf || (k_norm.buf && !pw)) return;
    launch_qsa_pool(c->stream, pp, pk, pw, pf, d, ratio, b0, b1, eps);
    cuda_ok(c, cudaGetLastError(), "qsa_pool launch");
}
extern "C" void qw_op_qsa_scores_pooled(qw_cmd c, qw_ref scores, qw_ref qn, qw_ref pool, int32_t rows, int32_t nq, int32_t d,
                                        int32_t ratio, int32_t base_pos, int32_t max_blocks) {
    if (!live(c) || !qsa_shape_ok(c, "qsa_scores_pooled", d, ratio, 64)) return;
    if (rows <= 0 || nq <= 0 || base_pos < 0 || max_blocks <= 0 || (base_pos + rows) / ratio > max_blocks) { cmd_fail(c, "qsa_scores_pooled: bad shape"); return; }
    const int32_t all = (base_pos + rows) / ratio;
    if (all == 0) return;
    float *ps = (float *)dev_range(c, scores, (size_t)rows * max_blocks * 4, true, 4);
    const float *pq = (const float *)dev_range(c, qn, (size_t)rows * nq * d * 4, false, 4);
    const float *pp = (const float *)dev_range(c, pool, (size_t)all * d * 4, false, 4);
    if (!ps || !pq || !pp) return;
    launch_qsa_scores(c->stream, ps, pq, pp, rows, nq, d, ratio, base_pos, max_blocks);
    cuda_ok(c, cudaGetLastError(), "qsa_scores_pooled launch");
}
extern "C" void qw_op_qsa_scores(qw_cmd c, qw_ref scores, qw_ref qn, qw_ref ikeys, qw_ref k_norm, qw_ref inv_freq, int32_t rows,
                                 int32_t nq, int32_t d, int32_t ratio, int32_t base_pos, int32_t rotary_dim, int32_t max_blocks, float eps) {
    if (!live(c) || !qsa_shape_ok(c, "qsa_scores", d, ratio, rotary_dim)) return;
    if (rows <= 0 || nq <= 0 || base_pos < 0 || max_blocks <= 0 || (base_pos + rows) / ratio > max_blocks) { cmd_fail(c, "qsa_scores: bad shape"); return; }
    const int32_t all = (base_pos + rows) / ratio;
    if (all == 0) return;
    float *ps = (float *)dev_range(c, scores, (size_t)rows * max_blocks * 4, true, 4);
    const float *pq = (const float *)dev_range(c, qn, (size_t)rows * nq * d * 4, false, 4);
    const float *pk = (const float *)dev_range(c, ikeys, (size_t)all * ratio * d * 4, false, 4);
    const uint16_t *pw = k_norm.buf ? (const uint16_t *)dev_range(c, k_norm, (size_t)d * 2, false, 2) : nullptr;
    const float *pf = (const float *)dev_range(c, inv_freq, 32 * 4, false, 4);
    if (!ps || !pq || !pk || !pf || (k_norm.buf && !pw)) return;
    // the block keys first (the same arithmetic as qw_op_qsa_pool, so both routes give identical scores), then the scores
    float *keys = (float *)cmd_scratch(c, (size_t)all * d * 4);
    if (!keys) return;
    launch_qsa_pool(c->stream, keys, pk, pw, pf, d, ratio, 0, all, eps);
    launch_qsa_scores(c->stream, ps, pq, keys, rows, nq, d, ratio, base_pos, max_blocks);
    cuda_ok(c, cudaGetLastError(), "qsa_scores launch");
}
extern "C" void qw_op_qsa_select(qw_cmd c, qw_ref mask, qw_ref list, qw_ref scores, int32_t rows, int32_t ratio, int32_t base_pos,
                                 int32_t block_topk, int32_t max_ctx, int32_t max_blocks) {
    if (!live(c)) return;
    if (rows <= 0 || ratio <= 0 || base_pos < 0 || block_topk < 0 || max_blocks <= 0 || (int64_t)base_pos + rows > max_ctx ||
        (base_pos + rows) / ratio > max_blocks || max_blocks > (1 << 20)) { cmd_fail(c, "qsa_select: bad shape"); return; }
    uint8_t *pm = (uint8_t *)dev_range(c, mask, (size_t)rows * max_ctx, true, 1);
    uint32_t *pl = (uint32_t *)dev_range(c, list, (size_t)rows * (1 + block_topk * ratio + ratio) * 4, true, 4);
    const float *ps = (const float *)dev_range(c, scores, (size_t)rows * max_blocks * 4, false, 4);
    if (!pm || !pl || !ps) return;
    launch_qsa_select(c->stream, pm, pl, ps, rows, ratio, base_pos, block_topk, max_ctx, max_blocks);
    cuda_ok(c, cudaGetLastError(), "qsa_select launch");
}

// Attention over listed positions only (the QSA mask as a list): the fp32 per-query kernel walks
// each row's list in `splits` slices, the merge combines them (and applies the gate).
static void attn_masked(qw_cmd c, qw_ref out, qw_ref gate, qw_ref q, qw_ref kcache, qw_ref vcache, qw_ref list, int32_t rows,
                        int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale,
                        int32_t block_topk, int32_t ratio) {
    if (!live(c)) return;
    if (head_dim != QW_HEAD_DIM) { fprintf(stderr, "qwasar: attention head_dim %d unsupported (kernel is built for 256)\n", head_dim); return; }
    if (!shape_ok(rows, q_heads, kv_heads, head_dim, max_ctx, base_pos) || block_topk < 0 || ratio <= 0) { cmd_fail(c, "attn_masked: bad shape"); return; }
    const int32_t cap = block_topk * ratio + ratio;               // qw_qsa_list_cap (qwasar_gpu.h:637-639)
    AttnSeq sq;
    memset(&sq, 0, sizeof sq);
    if (!resolve_cache(c, kcache, kv_heads, max_ctx, head_dim, base_pos + rows, false, false, &sq.kc, nullptr)) return;
    if (!resolve_cache(c, vcache, kv_heads, max_ctx, head_dim, base_pos + rows, false, false, &sq.vc, nullptr)) return;
    const size_t n = (size_t)rows * q_heads * head_dim * 4;
    sq.q = dev_range(c, q, n, false);
    void *po = dev_range(c, out, n, true);
    const void *pg = gate.buf ? dev_range(c, gate, n, false) : nullptr;
    const uint32_t *pl = (const uint32_t *)dev_range(c, list, (size_t)rows * (1 + cap) * 4, false, 4);
    if (!sq.q || !po || !pl || (gate.buf && !pg)) return;
    sq.rows = rows; sq.base_pos = base_pos; sq.key_lo = 0; sq.key_hi = base_pos + rows;
    if (g_tune_masked_tc && q_heads / kv_heads <= 16) {
        // one launch on a cluster where one can be placed; else tensor ops over the gathered rows with a partial per
        // 64 list entries, then the merge (and gate)
        if (g_tune_masked_tc == 1 && launch_attn_masked_cluster(c->stream, sq, q_heads, kv_heads, scale, pl, 1 + cap, (float *)po, (const float *)pg, 256)) {
            cuda_ok(c, cudaGetLastError(), "attn_masked launch");
            return;
        }
        const int chunks = attn_masked_chunks(cap);
        float *scr = (float *)cmd_scratch(c, attn_per_query_scratch_bytes(rows, q_heads, chunks));
        if (!scr) return;
        float *pstat = scr + (size_t)chunks * rows * q_heads * 256;
        launch_attn_masked_mma(c->stream, sq, q_heads, kv_heads, scale, pl, 1 + cap, scr, pstat);
        launch_merge_parts(c->stream, po, DT_F32, scr, pstat, pg, DT_F32, 256, rows * q_heads, chunks, nullptr, nullptr);
        cuda_ok(c, cudaGetLastError(), "attn_masked launch");
        return;
    }
    const int splits = attn_per_query_splits(rows, q_heads, cap);
    float *scr = (float *)cmd_scratch(c, attn_per_query_scratch_bytes(rows, q_heads, splits));
    if (!scr) return;
    float *pstat = scr + (size_t)splits * rows * q_heads * 256;
    launch_attn_per_query(c->stream, sq, q_heads, kv_heads, scale, scr, pstat, splits, pl, 1 + cap);
    launch_merge_parts(c->stream, po, DT_F32, scr, pstat, pg, DT_F32, 256, rows * q_heads, splits, nullptr, nullptr);
    cuda_ok(c, cudaGetLastError(), "attn_masked launch");
}
extern "C" void qw_op_attn_masked(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache, qw_ref list, int32_t rows,
                                  int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale,
                                  int32_t block_topk, int32_t ratio) {
    attn_masked(c, out, qw_ref{nullptr, 0}, q, kcache, vcache, list, rows, q_heads, kv_heads, head_dim, max_ctx, base_pos, scale, block_topk, ratio);
}
extern "C" void qw_op_attn_masked_gated(qw_cmd c, qw_ref out, qw_ref gate, qw_ref q, qw_ref kcache, qw_ref vcache, qw_ref list,
                                        int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_ctx,
                                        int32_t base_pos, float scale, int32_t block_topk, int32_t ratio) {
    if (!gate.buf) { if (c) cmd_fail(c, "attn_masked_gated: no gate"); return; }
    attn_masked(c, out, gate, q, kcache, vcache, list, rows, q_heads, kv_heads, head_dim, max_ctx, base_pos, scale, block_topk, ratio);
}

extern "C" bool qw_op_attn_decode_tensor(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache, int32_t rows,
                                         int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_ctx,
                                         int32_t base_pos, float scale) {
    if (!live(c) || !shape_ok(rows, q_heads, kv_heads, head_dim, max_ctx, base_pos)) return false;
    if (q_heads / kv_heads > 64) return false;            // rows beyond 64 / grouping are taken in chunks
    AttnArgs a = {out, q, qw_ref{nullptr, 0}, kcache, vcache, rows, base_pos};
    return attn_rows_split(c, &a, 1, q_heads, kv_heads, max_ctx, scale, DT_F32, DT_F32, DT_F32, 256);
}
extern "C" bool qw_op_attn_decode_split(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache, int32_t rows,
                                        int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_ctx,
                                        int32_t base_pos, float scale) {
    return qw_op_attn_decode_tensor(c, out, q, kcache, vcache, rows, q_heads, kv_heads, head_dim, max_ctx, base_pos, scale);
}

extern "C" bool qw_op_attn_prefill_as(qw_cmd c, bool half_form, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache,
                                      int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_ctx,
                                      int32_t base_pos, float scale) {
    (void)half_form;
    if (!live(c) || !shape_ok(rows, q_heads, kv_heads, head_dim, max_ctx, base_pos)) return false;
    const size_t n = (size_t)rows * q_heads * 256;
    void *op = dev_range(c, out, n * 4, true);
    if (!g_tune_prefill_tc || !attn_prefill_io_ok(op, DT_F32, nullptr, DT_F32, 256)) {
        if (q_heads / kv_heads > 64) return false;
        AttnArgs a = {out, q, qw_ref{nullptr, 0}, kcache, vcache, rows, base_pos};
        return attn_rows_split(c, &a, 1, q_heads, kv_heads, max_ctx, scale, DT_F32, DT_F32, DT_F32, 256);
    }
    const float *qp = (const float *)dev_range(c, q, n * 4, false);
    __nv_bfloat16 *qb = (__nv_bfloat16 *)cmd_scratch(c, n * 2);
    if (!qp || !op || !qb) return false;
    launch_f32_to_bf16(c->stream, qb, qp, (int64_t)n);
    return run_prefill(c, qb, op, DT_F32, nullptr, DT_F32, 256, kcache, vcache, rows, q_heads, kv_heads, max_ctx, base_pos, scale);
}
extern "C" bool qw_op_attn_prefill(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache, int32_t rows, int32_t q_heads,
                                   int32_t kv_heads, int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale) {
    return qw_op_attn_prefill_as(c, true, out, q, kcache, vcache, rows, q_heads, kv_heads, head_dim, max_ctx, base_pos, scale);
}

extern "C" void qw_op_attn(qw_cmd c, qw_ref out, qw_ref q, qw_ref kcache, qw_ref vcache, int32_t rows, int32_t q_heads,
                           int32_t kv_heads, int32_t head_dim, int32_t max_ctx, int32_t base_pos, float scale) {
    if (!live(c)) return;
    // one shape rule, no environment switches: many rows -> the tiled kernel, few -> split-KV
    if (rows >= 16 && qw_op_attn_prefill(c, out, q, kcache, vcache, rows, q_heads, kv_heads, head_dim, max_ctx, base_pos, scale)) return;
    if (rows < 16 && qw_op_attn_decode_tensor(c, out, q, kcache, vcache, rows, q_heads, kv_heads, head_dim, max_ctx, base_pos, scale)) return;
    if (c->failed) return;
    qw_op_attn_decode(c, out, q, kcache, vcache, rows, q_heads, kv_heads, head_dim, max_ctx, base_pos, scale);
}

// ---------------------------------------------------------------------------------------
// additive: fused node, batch, partials
// ---------------------------------------------------------------------------------------
namespace {

bool fused_check(int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t rotary_dim) {
    return rows > 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && head_dim == QW_HEAD_DIM && rotary_dim == 64;
}

struct FusedSeq { qw_ref out, qg, k, v, pos, kcache, vcache; int32_t base_pos; };

// pre-op for up to QW_MAX_SEQ sequences; q_out[i] receives each sequence's bf16 query.
// skip_q: the query heads are left alone (the attention kernel norms and rotates them itself) and
// q_out may be nullptr; cs_out != nullptr: the rotation angles' cos / sin of every row also go to
// cs_out[i] ([rows, 64] f32) -- the prefill kernel reads its angles from there.
bool run_preop(qw_cmd c, const FusedSeq *s, int n_seq, __nv_bfloat16 *const *q_out, qw_ref q_norm_w, qw_ref k_norm_w,
               qw_ref axis, qw_ref inv_freq, int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t max_ctx,
               float eps, int io, bool append, float *const *cs_out = nullptr, bool skip_q = false) {
    PreopParams p;
    memset(&p, 0, sizeof p);
    const size_t el = io == DT_BF16 ? 2 : 4;
    p.n_seq = n_seq; p.q_heads = q_heads; p.kv_heads = append ? kv_heads : 0; p.rotary_dim = 64; p.io_dtype = io; p.eps = eps;
    p.q_norm_w = q_norm_w.buf ? (const uint16_t *)dev_range(c, q_norm_w, 512, false) : nullptr;
    p.k_norm_w = k_norm_w.buf ? (const uint16_t *)dev_range(c, k_norm_w, 512, false) : nullptr;
    p.axis = (const uint8_t *)dev_range(c, axis, 32, false, 1);
    p.inv_freq = (const float *)dev_range(c, inv_freq, 128, false, 4);
    if (!p.axis || !p.inv_freq || (q_norm_w.buf && !p.q_norm_w) || (k_norm_w.buf && !p.k_norm_w)) return false;
    for (int i = 0; i < n_seq; i++) {
        PreopSeq &ps = p.seq[i];
        ps.qg = dev_range(c, s[i].qg, (size_t)rows * q_heads * 512 * el, false);
        ps.pos = (const int32_t *)dev_range(c, s[i].pos, (size_t)3 * rows * 4, false, 4);
        if (!ps.qg || !ps.pos) return false;
        if (append) {
            ps.k = dev_range(c, s[i].k, (size_t)rows * kv_heads * 256 * el, false);
            ps.v = dev_range(c, s[i].v, (size_t)rows * kv_heads * 256 * el, false);
            if (!ps.k || !ps.v) return false;
            if (!resolve_cache(c, s[i].kcache, kv_heads, max_ctx, QW_HEAD_DIM, s[i].base_pos + rows, true, true, &ps.kc, nullptr, 32, nullptr, s[i].base_pos)) return false;
            if (!resolve_cache(c, s[i].vcache, kv_heads, max_ctx, QW_HEAD_DIM, s[i].base_pos + rows, true, true, &ps.vc, nullptr, 32, nullptr, s[i].base_pos)) return false;
        }
        ps.q_out = q_out ? q_out[i] : nullptr;
        ps.cs_out = cs_out ? cs_out[i] : nullptr;
        ps.rows = rows; ps.base_pos = s[i].base_pos;
    }
    p.skip_q = skip_q || cs_out != nullptr;
    KTime kt = {nullptr, nullptr, "qw_attn_preop"};
    const bool timed = SH.time_kernels && cudaEventCreate(&kt.t0) == cudaSuccess && cudaEventCreate(&kt.t1) == cudaSuccess;
    if (timed) cudaEventRecord(kt.t0, c->stream);
    launch_preop(c->stream, p, rows);
    if (timed) { cudaEventRecord(kt.t1, c->stream); c->ktimes.push_back(kt); }
    return cuda_ok(c, cudaGetLastError(), "pre-op launch");
}

bool fused_batch(qw_cmd c, const FusedSeq *seqs, int n_seq, qw_ref q_norm_w, qw_ref k_norm_w, qw_ref axis, qw_ref inv_freq,
                 int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t max_ctx, float eps, float scale, int io) {
    const size_t el = io == DT_BF16 ? 2 : 4;
    const int gqa = q_heads / kv_heads;
    const int chunk_rows = std::max(1, 64 / gqa);
    for (int s0 = 0; s0 < n_seq; s0 += QW_MAX_SEQ) {
        const int ns = std::min(QW_MAX_SEQ, n_seq - s0);
        for (int i = 0; i < ns; i++)
            if ((int64_t)seqs[s0 + i].base_pos + rows > max_ctx || seqs[s0 + i].base_pos < 0) { cmd_fail(c, "fused attention: positions outside the cache"); return false; }
        if (rows * gqa > 64 && g_tune_prefill_tc) {
            // many rows: the tcgen05 kernel, one launch per sequence (operands that its tile maps
            // cannot describe, e.g. an output that is not 16-byte aligned, take the chunked path below)
            char *op[QW_MAX_SEQ];
            const char *gp[QW_MAX_SEQ];
            bool tiles_ok = true;
            for (int i = 0; i < ns; i++) {
                const FusedSeq &fs = seqs[s0 + i];
                op[i] = (char *)dev_range(c, fs.out, (size_t)rows * q_heads * 256 * el, true);
                gp[i] = (const char *)dev_range(c, fs.qg, (size_t)rows * q_heads * 512 * el, false);
                if (!op[i] || !gp[i]) return false;
                tiles_ok = tiles_ok && attn_prefill_io_ok(op[i], io, gp[i] + 256 * el, io, 512);
            }
            if (tiles_ok) {
                // scratch: per sequence the bf16 queries, or (bf16 rows: the kernel norms and rotates its
                // own query tiles, the pre-op only appends K and V) the rows' cos / sin in the same place
                const size_t q_bytes = (size_t)rows * q_heads * 256 * 2;
                char *scr = (char *)cmd_scratch(c, (size_t)ns * q_bytes);
                if (!scr) return false;
                __nv_bfloat16 *qo[QW_MAX_SEQ];
                float *cs[QW_MAX_SEQ];
                for (int i = 0; i < ns; i++) { qo[i] = reinterpret_cast<__nv_bfloat16 *>(scr + (size_t)i * q_bytes); cs[i] = reinterpret_cast<float *>(qo[i]); }
                const bool fuse_q = io == DT_BF16 && g_tune_prefill_fuse_q;
                const uint16_t *wq = q_norm_w.buf ? (const uint16_t *)dev_range(c, q_norm_w, 512, false) : nullptr;
                if (q_norm_w.buf && !wq) return false;
                if (!run_preop(c, seqs + s0, ns, qo, q_norm_w, k_norm_w, axis, inv_freq, rows, q_heads, kv_heads, max_ctx, eps, io, true,
                               fuse_q ? cs : nullptr)) return false;
                for (int i = 0; i < ns; i++) {
                    const FusedSeq &fs = seqs[s0 + i];
                    const bool ok = fuse_q
                        ? run_prefill(c, reinterpret_cast<const __nv_bfloat16 *>(gp[i]), op[i], io, gp[i] + 256 * el, io, 512, fs.kcache, fs.vcache,
                                      rows, q_heads, kv_heads, max_ctx, fs.base_pos, scale, cs[i], wq, eps)
                        : run_prefill(c, qo[i], op[i], io, gp[i] + 256 * el, io, 512, fs.kcache, fs.vcache, rows, q_heads, kv_heads,
                                      max_ctx, fs.base_pos, scale);
                    if (!ok) return false;
                }
                continue;
            }
        }
        // few rows (decode, verify), or rows in chunks: one kernel appends K and V, the split-KV
        // kernel norms and rotates the raw query rows itself and starts under the append
        if (!run_preop(c, seqs + s0, ns, nullptr, q_norm_w, k_norm_w, axis, inv_freq, rows, q_heads, kv_heads, max_ctx, eps, io, true,
                       nullptr, true)) return false;
        SplitBatch b;
        b.c = c;
        AttnParams &p = b.p;
        memset(&p, 0, sizeof p);
        p.q_heads = q_heads; p.kv_heads = kv_heads; p.gqa = gqa; p.q_dtype = io; p.out_dtype = io;
        p.gate_dtype = io; p.gate_stride = 512; p.scale = scale; p.mode = 0;
        p.q_raw = 1; p.eps = eps;
        p.q_norm_w = q_norm_w.buf ? (const uint16_t *)dev_range(c, q_norm_w, 512, false) : nullptr;
        p.axis = (const uint8_t *)dev_range(c, axis, 32, false, 1);
        p.inv_freq = (const float *)dev_range(c, inv_freq, 128, false, 4);
        if (!p.axis || !p.inv_freq || (q_norm_w.buf && !p.q_norm_w)) return false;
        b.early_next = !SH.time_kernels && g_tune_pdl;        // (event records between the kernels would serialise them anyway)
        for (int i = 0; i < ns; i++) {
            const FusedSeq &fs = seqs[s0 + i];
            KvLayer kc, vc;
            CUtensorMap km, vm;
            if (!resolve_cache(c, fs.kcache, kv_heads, max_ctx, QW_HEAD_DIM, fs.base_pos + rows, false, false, &kc, &km)) return false;
            if (!resolve_cache(c, fs.vcache, kv_heads, max_ctx, QW_HEAD_DIM, fs.base_pos + rows, false, false, &vc, &vm)) return false;
            char *op = (char *)dev_range(c, fs.out, (size_t)rows * q_heads * 256 * el, true);
            const char *gp = (const char *)dev_range(c, fs.qg, (size_t)rows * q_heads * 512 * el, false);
            const int32_t *pp = (const int32_t *)dev_range(c, fs.pos, (size_t)3 * rows * 4, false, 4);
            if (!op || !gp || !pp) return false;
            for (int r0 = 0; r0 < rows; r0 += chunk_rows) {
                AttnSeq sq;
                memset(&sq, 0, sizeof sq);
                const int rr = std::min(chunk_rows, rows - r0);
                sq.q = gp + (size_t)r0 * q_heads * 512 * el;               // the q half of each [q|gate] head
                sq.out = op + (size_t)r0 * q_heads * 256 * el;
                sq.gate = gp + ((size_t)r0 * q_heads * 512 + 256) * el;    // the gate half
                sq.pos = pp + r0; sq.pos_stride = rows;
                sq.kc = kc; sq.vc = vc;
                sq.rows = rr; sq.base_pos = fs.base_pos + r0;
                sq.fresh_pos = fs.base_pos;
                sq.key_lo = 0; sq.key_hi = fs.base_pos + r0 + rr;
                if (!b.add(sq, km, vm)) return false;
            }
        }
        if (!b.flush()) return false;
    }
    return true;
}

}  // namespace

extern "C" bool qw_op_attn_layer_fused(qw_cmd c, qw_ref out, qw_ref qg, qw_ref k, qw_ref v, qw_ref q_norm_w, qw_ref k_norm_w,
                                       qw_ref pos, qw_ref axis, qw_ref inv_freq, qw_ref kcache, qw_ref vcache, int32_t rows,
                                       int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t rotary_dim,
                                       int32_t max_ctx, int32_t base_pos, float eps, float scale, qw_dtype io) {
    if (!live(c) || !fused_check(rows, q_heads, kv_heads, head_dim, rotary_dim) || q_heads / kv_heads > 64) return false;
    FusedSeq s = {out, qg, k, v, pos, kcache, vcache, base_pos};
    return fused_batch(c, &s, 1, q_norm_w, k_norm_w, axis, inv_freq, rows, q_heads, kv_heads, max_ctx, eps, scale, (int)io);
}

extern "C" bool qw_op_attn_layer_fused_batch(qw_cmd c, int32_t n_seq, const qw_ref *out, const qw_ref *qg, const qw_ref *k,
                                             const qw_ref *v, qw_ref q_norm_w, qw_ref k_norm_w, const qw_ref *pos, qw_ref axis,
                                             qw_ref inv_freq, const qw_ref *kcache, const qw_ref *vcache,
                                             const int32_t *base_pos, int32_t rows, int32_t q_heads, int32_t kv_heads,
                                             int32_t head_dim, int32_t rotary_dim, int32_t max_ctx, float eps, float scale,
                                             qw_dtype io) {
    if (!live(c) || n_seq <= 0 || !fused_check(rows, q_heads, kv_heads, head_dim, rotary_dim) || q_heads / kv_heads > 64) return false;
    std::vector<FusedSeq> s((size_t)n_seq);
    for (int i = 0; i < n_seq; i++) s[(size_t)i] = FusedSeq{out[i], qg[i], k[i], v[i], pos[i], kcache[i], vcache[i], base_pos[i]};
    return fused_batch(c, s.data(), n_seq, q_norm_w, k_norm_w, axis, inv_freq, rows, q_heads, kv_heads, max_ctx, eps, scale, (int)io);
}

extern "C" bool qw_op_attn_batch(qw_cmd c, int32_t n_seq, const qw_ref *out, const qw_ref *q, const qw_ref *kcache,
                                 const qw_ref *vcache, const int32_t *base_pos, int32_t rows, int32_t q_heads, int32_t kv_heads,
                                 int32_t head_dim, int32_t max_ctx, float scale, qw_dtype io) {
    if (!live(c) || n_seq <= 0) return false;
    std::vector<AttnArgs> a((size_t)n_seq);
    for (int i = 0; i < n_seq; i++) {
        if (!shape_ok(rows, q_heads, kv_heads, head_dim, max_ctx, base_pos[i])) return false;
        a[(size_t)i] = AttnArgs{out[i], q[i], qw_ref{nullptr, 0}, kcache[i], vcache[i], rows, base_pos[i]};
    }
    if (q_heads / kv_heads > 64) return false;
    return attn_rows_split(c, a.data(), n_seq, q_heads, kv_heads, max_ctx, scale, (int)io, (int)io, DT_F32, 256);
}

extern "C" bool qw_op_attn_preop(qw_cmd c, qw_ref q_out, qw_ref qg, qw_ref k, qw_ref v, qw_ref q_norm_w, qw_ref k_norm_w,
                                 qw_ref pos, qw_ref axis, qw_ref inv_freq, qw_ref kcache, qw_ref vcache, int32_t rows,
                                 int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t rotary_dim, int32_t max_ctx,
                                 int32_t base_pos, float eps, qw_dtype io, bool append) {
    if (!live(c) || !fused_check(rows, q_heads, kv_heads, head_dim, rotary_dim)) return false;
    if (append && (base_pos < 0 || (int64_t)base_pos + rows > max_ctx)) return false;
    __nv_bfloat16 *qo = (__nv_bfloat16 *)dev_range(c, q_out, (size_t)rows * q_heads * 256 * 2, true);
    if (!qo) return false;
    FusedSeq s = {qw_ref{nullptr, 0}, qg, k, v, pos, kcache, vcache, base_pos};
    return run_preop(c, &s, 1, &qo, q_norm_w, k_norm_w, axis, inv_freq, rows, q_heads, kv_heads, max_ctx, eps, (int)io, append);
}

extern "C" bool qw_op_attn_partial(qw_cmd c, qw_ref pacc, qw_ref pstat, qw_ref q, qw_ref kcache, qw_ref vcache, int32_t rows,
                                   int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_ctx, int32_t base_pos,
                                   int32_t key_lo, int32_t key_hi, float scale, qw_dtype q_dtype) {
    if (!live(c) || !shape_ok(rows, q_heads, kv_heads, head_dim, max_ctx, base_pos)) return false;
    const int gqa = q_heads / kv_heads;
    if (rows * gqa > 64 || key_lo < 0) return false;
    key_hi = std::min(key_hi, base_pos + rows);
    // an empty range needs no alignment (a trailing shard of a short sequence starts where the keys end)
    if (key_hi > key_lo && (key_lo & 63)) return false;
    const size_t n_rh = (size_t)rows * q_heads;
    float *pa = (float *)dev_range(c, pacc, n_rh * 256 * 4, true), *ps = (float *)dev_range(c, pstat, n_rh * 2 * 4, true);
    if (!pa || !ps) return false;
    if (key_hi <= key_lo) {
        // nothing of this range is visible: an empty partial (sum 0 drops out of the merge)
        cuda_ok(c, cudaMemsetAsync(pa, 0, n_rh * 256 * 4, c->stream), "memset");
        cuda_ok(c, cudaMemsetAsync(ps, 0, n_rh * 2 * 4, c->stream), "memset");
        return !c->failed;
    }
    AttnParams p;
    memset(&p, 0, sizeof p);
    p.n_seq = 1; p.q_heads = q_heads; p.kv_heads = kv_heads; p.gqa = gqa; p.q_dtype = (int)q_dtype; p.out_dtype = DT_F32;
    p.gate_dtype = DT_F32; p.gate_stride = 256; p.scale = scale; p.mode = 1;
    AttnSeq &sq = p.seq[0];
    if (!resolve_cache(c, kcache, kv_heads, max_ctx, head_dim, key_hi, false, false, &sq.kc, &p.maps[0])) return false;
    if (!resolve_cache(c, vcache, kv_heads, max_ctx, head_dim, key_hi, false, false, &sq.vc, &p.maps[1])) return false;
    sq.kmap = 0; sq.vmap = 1;
    sq.q = dev_range(c, q, n_rh * 256 * (q_dtype == QW_BF16 ? 2 : 4), false);
    if (!sq.q) return false;
    sq.rows = rows; sq.base_pos = base_pos; sq.key_lo = key_lo; sq.key_hi = key_hi;
    p.comb_acc = pa;          // the merge leaves the one combined partial per (row, head) here
    p.comb_stat = ps;
    return run_split(c, p, rows);
}

extern "C" void qw_op_attn_merge(qw_cmd c, qw_ref out, qw_ref pacc, qw_ref pstat, qw_ref gate, int32_t rows, int32_t q_heads,
                                 int32_t head_dim, int32_t parts, int32_t gate_stride, qw_dtype out_dtype, qw_dtype gate_dtype,
                                 int64_t part_stride) {
    if (!live(c) || rows <= 0 || q_heads <= 0 || parts <= 0 || head_dim != QW_HEAD_DIM || part_stride < 0) return;
    const size_t n_rh = (size_t)rows * q_heads;
    const size_t a_stride = part_stride ? (size_t)part_stride : n_rh * 256, s_stride = part_stride ? (size_t)part_stride : n_rh * 2;
    const float *pa = (const float *)dev_range(c, pacc, ((size_t)(parts - 1) * a_stride + n_rh * 256) * 4, false);
    const float *ps = (const float *)dev_range(c, pstat, ((size_t)(parts - 1) * s_stride + n_rh * 2) * 4, false);
    void *po = dev_range(c, out, n_rh * 256 * (out_dtype == QW_BF16 ? 2 : 4), true);
    const size_t g_el = gate_dtype == QW_BF16 ? 2 : 4;
    const void *pg = gate.buf ? dev_range(c, gate, ((n_rh - 1) * gate_stride + 256) * g_el, false) : nullptr;
    if (!pa || !ps || !po || (gate.buf && !pg)) return;
    launch_merge_parts(c->stream, po, (int)out_dtype, pa, ps, pg, (int)gate_dtype, gate_stride, (int)n_rh, parts, nullptr, nullptr,
                       a_stride, s_stride);
    cuda_ok(c, cudaGetLastError(), "merge launch");
}

// ---------------------------------------------------------------------------------------
// additive: the exchange of partials between the GPUs that hold one sequence
// ---------------------------------------------------------------------------------------
struct qw_xchg_s {
    int device, n_ranks, rank, max_rh;
    void *base;                 // one allocation: the gather buffer, then the flags
    size_t gather_bytes, flags_bytes;
    float *peer_gather[8];      // every rank's buffer as this process addresses it ([rank] = own)
    int *peer_flags[8];
    void *opened[8];            // mappings of other processes' buffers, closed by qw_xchg_free
    int epoch;
    int64_t timeout_ns;
};

extern "C" qw_xchg qw_xchg_create(int32_t n_ranks, int32_t rank, int32_t max_rows_heads) {
    if (!G.up) { set_error("qw_xchg_create before qw_gpu_init"); return nullptr; }
    if (n_ranks < 1 || n_ranks > 8 || rank < 0 || rank >= n_ranks || max_rows_heads <= 0) { set_error("qw_xchg_create: 1 to 8 ranks, a rank among them, a positive row count"); return nullptr; }
    qw_xchg x = new qw_xchg_s();
    memset(x, 0, sizeof *x);
    x->device = G.device; x->n_ranks = n_ranks; x->rank = rank; x->max_rh = max_rows_heads;
    x->gather_bytes = (size_t)2 * n_ranks * max_rows_heads * QW_XCHG_REC * sizeof(float);
    x->flags_bytes = (size_t)2 * n_ranks * max_rows_heads * sizeof(int);
    if (cudaMalloc(&x->base, x->gather_bytes + x->flags_bytes) != cudaSuccess) { set_error("qw_xchg_create: out of device memory"); cudaGetLastError(); delete x; return nullptr; }
    cudaMemset(x->base, 0, x->gather_bytes + x->flags_bytes);       // no flag shows an epoch yet
    cudaDeviceSynchronize();
    x->peer_gather[rank] = (float *)x->base;
    x->peer_flags[rank] = (int *)((char *)x->base + x->gather_bytes);
    x->timeout_ns = (int64_t)2000 * 1000 * 1000;
    return x;
}

extern "C" void qw_xchg_free(qw_xchg x) {
    if (!x) return;
    use_device(x->device);
    cudaDeviceSynchronize();
    for (int i = 0; i < 8; i++) if (x->opened[i]) cudaIpcCloseMemHandle(x->opened[i]);
    cudaFree(x->base);
    delete x;
}

extern "C" size_t qw_xchg_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

extern "C" bool qw_xchg_export(qw_xchg x, void *handle) {
    if (!x || !handle) return false;
    use_device(x->device);
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, x->base) != cudaSuccess) { set_error("qw_xchg_export: %s", cudaGetErrorString(cudaGetLastError())); return false; }
    memcpy(handle, &h, sizeof h);
    return true;
}

extern "C" bool qw_xchg_attach(qw_xchg x, int32_t peer_rank, const void *handle) {
    if (!x || !handle || peer_rank < 0 || peer_rank >= x->n_ranks || peer_rank == x->rank) { set_error("qw_xchg_attach: bad rank"); return false; }
    use_device(x->device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void *p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        set_error("qw_xchg_attach: cannot map rank %d's buffer: %s", peer_rank, cudaGetErrorString(cudaGetLastError()));
        return false;
    }
    if (x->opened[peer_rank]) cudaIpcCloseMemHandle(x->opened[peer_rank]);
    x->opened[peer_rank] = p;
    x->peer_gather[peer_rank] = (float *)p;
    x->peer_flags[peer_rank] = (int *)((char *)p + x->gather_bytes);
    return true;
}

extern "C" bool qw_xchg_attach_local(qw_xchg x, int32_t peer_rank, qw_xchg peer) {
    if (!x || !peer || peer_rank < 0 || peer_rank >= x->n_ranks || peer_rank == x->rank || peer->rank != peer_rank ||
        peer->n_ranks != x->n_ranks || peer->max_rh != x->max_rh) { set_error("qw_xchg_attach_local: the two ends do not match"); return false; }
    x->peer_gather[peer_rank] = (float *)peer->base;
    x->peer_flags[peer_rank] = (int *)((char *)peer->base + peer->gather_bytes);
    return true;
}

extern "C" void qw_xchg_set_timeout_ms(qw_xchg x, int32_t ms) { if (x && ms > 0) x->timeout_ns = (int64_t)ms * 1000 * 1000; }

// One exchange round for n_seq sequences of equal shape.  Sequences whose range on this rank is
// empty publish empty records from a launch of the second kernel alone; the others go through the
// split-KV kernel first.  Slot numbers follow the sequence's place in the call on every rank.
static bool attn_exchange(qw_cmd c, qw_xchg x, int32_t phase, int32_t n_seq, const qw_ref *out, const qw_ref *gate, const qw_ref *q,
                          const qw_ref *kcache, const qw_ref *vcache, const int32_t *base_pos, const int32_t *key_lo,
                          const int32_t *key_hi, int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                          int32_t max_ctx, float scale, qw_dtype q_dtype, qw_dtype out_dtype, qw_dtype gate_dtype,
                          int32_t gate_stride) {
    if (!live(c) || !x || phase < 0 || phase > 2 || n_seq <= 0 || n_seq > QW_MAX_SEQ) return false;
    if (rows <= 0 || kv_heads <= 0 || q_heads <= 0 || q_heads % kv_heads || head_dim != QW_HEAD_DIM) return false;
    const int gqa = q_heads / kv_heads;
    const size_t n_rh = (size_t)rows * q_heads;
    if (rows * gqa > 64 || (size_t)n_seq * n_rh > (size_t)x->max_rh || x->device != c->device) {
        cmd_fail(c, "attn_exchange: shape does not fit the exchange (rows * grouping <= 64, sequences * rows * q_heads <= %d, same device)", x->max_rh);
        return false;
    }
    for (int i = 0; i < x->n_ranks; i++)
        if (!x->peer_gather[i]) { cmd_fail(c, "attn_exchange: rank %d was never attached", i); return false; }
    AttnParams base;
    memset(&base, 0, sizeof base);
    base.q_heads = q_heads; base.kv_heads = kv_heads; base.gqa = gqa; base.q_dtype = (int)q_dtype; base.out_dtype = (int)out_dtype;
    base.gate_dtype = (int)gate_dtype; base.gate_stride = gate_stride; base.scale = scale;
    base.mode = phase == 0 ? 2 : phase == 1 ? 3 : 4;
    if (phase != 2) x->epoch++;               // a new round: every rank must make the same calls in the same order
    for (int i = 0; i < x->n_ranks; i++) { base.x.gather[i] = x->peer_gather[i]; base.x.flags[i] = x->peer_flags[i]; }
    base.x.n_ranks = x->n_ranks; base.x.rank = x->rank; base.x.max_rh = x->max_rh; base.x.epoch = x->epoch;
    base.x.timeout_ns = x->timeout_ns;
    // two launches at most: the sequences with keys here, and the ones without (or, in phase 2, all)
    for (int pass = 0; pass < 2; pass++) {
        AttnParams p = base;
        int slot0[QW_MAX_SEQ];
        int n = 0, n_maps = 0;
        for (int i = 0; i < n_seq; i++) {
            if (!shape_ok(rows, q_heads, kv_heads, head_dim, max_ctx, base_pos[i]) || key_lo[i] < 0) return false;
            const int hi = std::min(key_hi[i], base_pos[i] + rows);
            const bool empty = hi <= key_lo[i] || phase == 2;
            if (empty != (pass == 1)) continue;
            if (!empty && (key_lo[i] & 63)) return false;
            AttnSeq &sq = p.seq[n];
            sq.rows = rows; sq.base_pos = base_pos[i]; sq.key_lo = empty ? 0 : key_lo[i]; sq.key_hi = empty ? 1 : hi;
            if (phase != 1) {
                const size_t g_el = gate_dtype == QW_BF16 ? 2 : 4;
                sq.out = dev_range(c, out[i], n_rh * 256 * (out_dtype == QW_BF16 ? 2 : 4), true);
                sq.gate = gate && gate[i].buf ? dev_range(c, gate[i], ((n_rh - 1) * gate_stride + 256) * g_el, false) : nullptr;
                if (!sq.out || (gate && gate[i].buf && !sq.gate)) return false;
            }
            if (!empty) {
                CUtensorMap km, vm;
                if (!resolve_cache(c, kcache[i], kv_heads, max_ctx, head_dim, hi, false, false, &sq.kc, &km)) return false;
                if (!resolve_cache(c, vcache[i], kv_heads, max_ctx, head_dim, hi, false, false, &sq.vc, &vm)) return false;
                int k = -1, v = -1;
                for (int m = 0; m < n_maps; m++) { if (!memcmp(&p.maps[m], &km, sizeof km)) k = m; if (!memcmp(&p.maps[m], &vm, sizeof vm)) v = m; }
                if (k < 0 && n_maps < QW_MAX_MAPS) { p.maps[n_maps] = km; k = n_maps++; }
                if (v < 0 && !memcmp(&km, &vm, sizeof km)) v = k;
                if (v < 0 && n_maps < QW_MAX_MAPS) { p.maps[n_maps] = vm; v = n_maps++; }
                if (k < 0 || v < 0) { cmd_fail(c, "attn_exchange: the sequences' caches lie in more than %d buffers or pools", QW_MAX_MAPS); return false; }
                sq.kmap = (uint8_t)k; sq.vmap = (uint8_t)v;
                sq.q = dev_range(c, q[i], n_rh * 256 * (q_dtype == QW_BF16 ? 2 : 4), false);
                if (!sq.q) return false;
            }
            slot0[n++] = i * rows;
        }
        if (!n) continue;
        p.n_seq = n;
        p.x.empty = pass;
        plan_split(p);
        for (int i = 0; i < n; i++) p.seq[i].row_slot0 = slot0[i];
        if (pass == 1) {
            p.status = cmd_status(c);
            launch_attn_merge(c->stream, p, rows);
            if (!cuda_ok(c, cudaGetLastError(), "exchange launch")) return false;
        } else {
            float *scr = (float *)cmd_scratch(c, attn_split_scratch_bytes(p, rows));
            if (!scr || !launch_split_merge(c, p, rows, scr)) return false;
        }
    }
    return true;
}

extern "C" bool qw_op_attn_exchange(qw_cmd c, qw_xchg x, int32_t phase, qw_ref out, qw_ref gate, qw_ref q, qw_ref kcache, qw_ref vcache,
                                    int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_ctx,
                                    int32_t base_pos, int32_t key_lo, int32_t key_hi, float scale, qw_dtype q_dtype,
                                    qw_dtype out_dtype, qw_dtype gate_dtype, int32_t gate_stride) {
    return attn_exchange(c, x, phase, 1, &out, &gate, &q, &kcache, &vcache, &base_pos, &key_lo, &key_hi, rows, q_heads, kv_heads,
                         head_dim, max_ctx, scale, q_dtype, out_dtype, gate_dtype, gate_stride);
}

extern "C" bool qw_op_attn_exchange_batch(qw_cmd c, qw_xchg x, int32_t phase, int32_t n_seq, const qw_ref *out, const qw_ref *gate,
                                          const qw_ref *q, const qw_ref *kcache, const qw_ref *vcache, const int32_t *base_pos,
                                          const int32_t *key_lo, const int32_t *key_hi, int32_t rows, int32_t q_heads,
                                          int32_t kv_heads, int32_t head_dim, int32_t max_ctx, float scale, qw_dtype q_dtype,
                                          qw_dtype out_dtype, qw_dtype gate_dtype, int32_t gate_stride) {
    if (!out || !q || !kcache || !vcache || !base_pos || !key_lo || !key_hi) return false;
    return attn_exchange(c, x, phase, n_seq, out, gate, q, kcache, vcache, base_pos, key_lo, key_hi, rows, q_heads, kv_heads,
                         head_dim, max_ctx, scale, q_dtype, out_dtype, gate_dtype, gate_stride);
}
