// qw_attn_decode_noalloc: split-KV decode attention for callers that may not allocate.
//
// Some embedders of this library hand every byte of device memory to their own pool at start-up,
// or run their decode loop in a phase where cudaMalloc is off limits because it synchronises the
// whole device (a serving loop with other streams in flight, a real-time budget).  The regular
// entry points take their partial-softmax scratch from a grow-on-demand pool, so their first call
// at a new size allocates.  This one never does: its scratch is a fixed array that is part of the
// loaded module, it takes raw device pointers for everything else, and it neither needs nor
// touches the state qw_gpu_init sets up.
#include "../../include/qwasar_cuda.h"
#include "qw_kernels.h"

#include <cstdio>
#include <cstring>

using namespace qw;

// The scratch: every GPU that loads this library carries these 4 MiB until the process exits.
// It holds one (max, sum, acc[256]) partial per (CTA or kv head, query row) -- 258 floats each.
#define QW_NOALLOC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) unsigned char g_noalloc_scratch[QW_NOALLOC_SCRATCH_BYTES];
// Where this entry point's kernels leave a status code when one of their bounded waits runs out
// (the regular ops report through their command buffer; this one has none).  0 = nothing happened.
static __device__ int g_noalloc_status;

namespace {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr int MAX_DEVICES = 64;
struct PerDevice {
    bool ready;
    float *scratch;      // device address of g_noalloc_scratch on that device
    int *status;         // device address of g_noalloc_status on that device
    int sms;
};
PerDevice g_dev[MAX_DEVICES];
PFN_encodeTiled g_encode = nullptr;

bool fail(char *err, size_t cap, const char *msg) {
    if (err && cap) snprintf(err, cap, "%s", msg);
    return false;
}

// First call on a device: resolve the array's device address.  In host code the name
// g_noalloc_scratch is only a handle for the symbol; the address a kernel can use comes from
// cudaGetSymbolAddress, asked with that device current.
bool setup_device(int dev, char *err, size_t cap) {
    if (dev < 0 || dev >= MAX_DEVICES) return fail(err, cap, "qw_attn_decode_noalloc: device index out of range");
    PerDevice &d = g_dev[dev];
    if (d.ready) return true;
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
        char msg[200];
        snprintf(msg, sizeof msg, "qw_attn_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        return fail(err, cap, msg);
    }
    if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || d.sms <= 0)
        return fail(err, cap, "qw_attn_decode_noalloc: cannot read the SM count");
    if (!g_encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !fn)
            return fail(err, cap, "qw_attn_decode_noalloc: driver lacks cuTensorMapEncodeTiled");
        g_encode = reinterpret_cast<PFN_encodeTiled>(fn);
    }
    void *st = nullptr;
    e = cudaGetSymbolAddress(&st, g_noalloc_status);
    if (e != cudaSuccess || !st) return fail(err, cap, "qw_attn_decode_noalloc: cudaGetSymbolAddress failed for the status word");
    d.scratch = reinterpret_cast<float *>(ptr);
    d.status = reinterpret_cast<int *>(st);
    d.ready = true;
    return true;
}

bool rows_map(CUtensorMap *m, const void *base, uint64_t rows) {
    cuuint64_t dims[2] = {QW_HEAD_DIM, rows};
    cuuint64_t strides[1] = {QW_HEAD_DIM * 2};
    cuuint32_t box[2] = {64, 32};
    cuuint32_t estr[2] = {1, 1};
    return g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" size_t qw_attn_decode_noalloc_scratch_bytes(void) { return QW_NOALLOC_SCRATCH_BYTES; }

extern "C" bool qw_attn_decode_noalloc(void *out, const void *q, const void *gate, const void *kcache, const void *vcache,
                                       int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                                       int32_t max_ctx, int32_t base_pos, float scale, qw_dtype io, void *cuda_stream,
                                       char *err, size_t errcap) {
    if (!out || !q || !kcache || !vcache) return fail(err, errcap, "qw_attn_decode_noalloc: null operand");
    if (head_dim != QW_HEAD_DIM) return fail(err, errcap, "qw_attn_decode_noalloc: head_dim must be 256");
    if (rows <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || base_pos < 0 || (int64_t)base_pos + rows > max_ctx)
        return fail(err, errcap, "qw_attn_decode_noalloc: bad shape or positions outside the cache");
    const int gqa = q_heads / kv_heads;
    if (rows * gqa > 16)
        return fail(err, errcap, "qw_attn_decode_noalloc: rows * (q_heads / kv_heads) exceeds 16, the limit of this entry point");
    if (((uintptr_t)kcache | (uintptr_t)vcache) & 127) return fail(err, errcap, "qw_attn_decode_noalloc: caches must be 128-byte aligned");
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)gate) & 15) return fail(err, errcap, "qw_attn_decode_noalloc: q, out and gate must be 16-byte aligned");
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(err, errcap, "qw_attn_decode_noalloc: no current CUDA device");
    if (!setup_device(dev, err, errcap)) return false;

    AttnParams p;
    memset(&p, 0, sizeof p);
    p.n_seq = 1; p.q_heads = q_heads; p.kv_heads = kv_heads; p.gqa = gqa;
    p.q_dtype = (int)io; p.out_dtype = (int)io; p.gate_dtype = (int)io; p.gate_stride = 256; p.scale = scale; p.mode = 0;
    AttnSeq &s = p.seq[0];
    s.q = q; s.out = out; s.gate = gate;
    s.kc.base = (__nv_bfloat16 *)kcache; s.kc.max_ctx = max_ctx;
    s.vc.base = (__nv_bfloat16 *)vcache; s.vc.max_ctx = max_ctx;
    s.rows = rows; s.base_pos = base_pos; s.key_lo = 0; s.key_hi = base_pos + rows;
    s.tile0 = 0; s.n_tiles = (s.key_hi + 31) / 32; s.cum_tiles = 0; s.row_slot0 = 0;
    p.total_tiles = s.n_tiles * kv_heads;
    p.n_cta = p.total_tiles < g_dev[dev].sms ? p.total_tiles : g_dev[dev].sms;
    if (p.n_cta > 256) p.n_cta = 256;                       // the merge kernel reads one partial per thread of 256
    const size_t need = attn_split_scratch_bytes(p, rows);
    if (need > QW_NOALLOC_SCRATCH_BYTES) {
        char msg[200];
        snprintf(msg, sizeof msg, "qw_attn_decode_noalloc: this shape needs %zu bytes of scratch, the built-in array holds %u",
                 need, QW_NOALLOC_SCRATCH_BYTES);
        return fail(err, errcap, msg);
    }
    s.kmap = 0; s.vmap = 1;
    if (!rows_map(&p.maps[0], kcache, (uint64_t)kv_heads * max_ctx) || !rows_map(&p.maps[1], vcache, (uint64_t)kv_heads * max_ctx))
        return fail(err, errcap, "qw_attn_decode_noalloc: cuTensorMapEncodeTiled failed");
    // partial slots first, their (max, sum) pairs after them -- the layout the kernels expect.  Nothing
    // in the array has to start at zero: every slot the merge reads was written by this call's launch.
    const size_t part_rows = (size_t)attn_split_slots(p) * 16 + (size_t)rows * q_heads;
    p.pacc = g_dev[dev].scratch;
    p.pstat = g_dev[dev].scratch + part_rows * 256;
    p.status = g_dev[dev].status;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    cudaGetLastError();        // an error left behind by earlier, unrelated work is not this call's
    launch_attn_split(stream, p, rows);
    launch_attn_merge(stream, p, rows);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        char msg[200];
        snprintf(msg, sizeof msg, "qw_attn_decode_noalloc: launch failed: %s", cudaGetErrorString(e));
        return fail(err, errcap, msg);
    }
    return true;
}

// The status word of the calling thread's current device, and cleared: 0 when every kernel of the
// earlier calls ran to its end, else the code of the wait that gave up (1 TMA load, 2 pipeline
// stage, 4 unmapped page).  Blocks until the device is idle of this module's copies only in the
// sense of cudaMemcpyFromSymbol: synchronise the streams of the calls first.  Allocates nothing.
extern "C" int32_t qw_attn_decode_noalloc_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_noalloc_status, sizeof v) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_noalloc_status, &zero, sizeof zero);
    return v;
}
