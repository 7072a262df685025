"""ctypes binding of libqwasar_cuda.so: the reference's qw_* names, argument
order and error behaviour (qwasar_gpu.h), plus the additive entry points.

Nothing here computes: every method forwards to the C ABI.  Loading fails with
an exception when the library has not been built, and `Backend()` raises when
qw_gpu_init reports no usable device."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("QWASAR_CUDA_LIB") or os.path.join(HERE, "libqwasar_cuda.so")   # (the override: for comparing two builds)
HEADER = os.path.join(os.path.dirname(HERE), "include", "qwasar_cuda.h")

F32, BF16 = 0, 1


class QwRef(C.Structure):
    """qw_ref: {qw_buf buf; size_t off;} passed by value (qwasar_gpu.h:45-52)."""
    _fields_ = [("buf", C.c_void_p), ("off", C.c_size_t)]


NULL_REF = QwRef(None, 0)
_i32, _f32, _vp, _sz, _b = C.c_int32, C.c_float, C.c_void_p, C.c_size_t, C.c_bool
_ATTN = [_vp, QwRef, QwRef, QwRef, QwRef, _i32, _i32, _i32, _i32, _i32, _i32, _f32]

# name -> (restype, argtypes); every symbol include/qwasar_cuda.h declares
SIGNATURES = {
    "qw_gpu_init": (_b, [C.c_char_p, _sz]),
    "qw_gpu_shutdown": (None, []),
    "qw_gpu_name": (C.c_char_p, []),
    "qw_gpu_working_set_limit": (C.c_uint64, []),
    "qw_gpu_max_buffer_length": (C.c_uint64, []),
    "qw_buf_wrap": (_vp, [_vp, _sz]),
    "qw_buf_alloc": (_vp, [_sz]),
    "qw_buf_free": (None, [_vp]),
    "qw_buf_contents": (_vp, [_vp]),
    "qw_buf_length": (_sz, [_vp]),
    "qw_cmd_begin": (_vp, []),
    "qw_cmd_commit": (None, [_vp]),
    "qw_cmd_wait": (None, [_vp]),
    "qw_cmd_flush": (None, [_vp]),
    "qw_cmd_parallel": (None, [_vp, _b]),
    "qw_cmd_free": (None, [_vp]),
    "qw_cmd_error": (C.c_char_p, [_vp]),
    "qw_prof_enabled": (_b, []),
    "qw_cmd_mark": (None, [_vp, C.c_char_p]),
    "qw_prof_report": (None, [_vp, C.c_long]),      # FILE *out, long tokens
    "qw_prof_reset": (None, []),
    "qw_op_split_heads2": (None, [_vp, QwRef, QwRef, QwRef, _i32, _i32, _i32]),
    "qw_op_rms_norm": (None, [_vp, QwRef, QwRef, QwRef, _i32, _i32, _f32, _f32]),
    "qw_op_rope_partial": (None, [_vp, QwRef, QwRef, QwRef, QwRef, _i32, _i32, _i32, _i32]),
    "qw_rope_tables": (None, [_vp, _vp, _i32, _f32, _vp]),
    "qw_op_mul_sigmoid": (None, [_vp, QwRef, QwRef, _i32]),
    "qw_op_slice_rows": (None, [_vp, QwRef, QwRef, _i32, _i32, _i32, _i32]),
    "qw_op_kv_write": (None, [_vp, QwRef, QwRef, QwRef, QwRef, _i32, _i32, _i32, _i32, _i32]),
    "qw_op_attn_decode": (None, _ATTN),
    "qw_op_attn_prefill": (_b, _ATTN),
    "qw_op_attn_prefill_as": (_b, [_vp, _b] + _ATTN[1:]),
    "qw_op_attn_decode_split": (_b, _ATTN),
    "qw_op_attn_decode_tensor": (_b, _ATTN),
    "qw_op_attn": (None, _ATTN),
    "qw_op_attn_masked": (None, [_vp, QwRef, QwRef, QwRef, QwRef, QwRef] + [_i32] * 6 + [_f32, _i32, _i32]),
    "qw_op_attn_masked_gated": (None, [_vp, QwRef, QwRef, QwRef, QwRef, QwRef, QwRef] + [_i32] * 6 + [_f32, _i32, _i32]),
    "qw_op_qsa_scores": (None, [_vp, QwRef, QwRef, QwRef, QwRef, QwRef] + [_i32] * 7 + [_f32]),
    "qw_op_qsa_pool": (None, [_vp, QwRef, QwRef, QwRef, QwRef] + [_i32] * 5 + [_f32]),
    "qw_op_qsa_scores_pooled": (None, [_vp, QwRef, QwRef, QwRef] + [_i32] * 6),
    "qw_op_qsa_select": (None, [_vp, QwRef, QwRef, QwRef] + [_i32] * 6),
    "qw_op_qmat_q4": (None, [_vp, QwRef, QwRef, QwRef, QwRef, QwRef] + [_i32] * 4),
    "qw_op_qmv_q4": (None, [_vp, QwRef, QwRef, QwRef, QwRef, QwRef] + [_i32] * 4),
    "qw_op_qmm_q4": (None, [_vp, QwRef, QwRef, QwRef, QwRef, QwRef] + [_i32] * 4),
    "qw_op_qmv_q4_multi": (_b, [_vp, QwRef, _i32, _i32, _i32, _vp]),
    "qw_gpu_device_count": (_i32, []),
    "qw_gpu_init_multi": (_b, [_i32, C.c_char_p, _sz]),
    "qw_gpu_select": (_b, [_i32]),
    "qw_gpu_current": (_i32, []),
    "qw_kv_pool_alloc": (_vp, [_sz, C.c_uint32]),
    "qw_kv_arena_alloc_in": (_vp, [_vp, _i32, _i32, _i32, _i32]),
    "qw_kv_pool_bytes_committed": (C.c_int64, [_vp]),
    "qw_xchg_create": (_vp, [_i32, _i32, _i32]),
    "qw_xchg_free": (None, [_vp]),
    "qw_xchg_handle_bytes": (_sz, []),
    "qw_xchg_export": (_b, [_vp, _vp]),
    "qw_xchg_attach": (_b, [_vp, _i32, _vp]),
    "qw_xchg_attach_local": (_b, [_vp, _i32, _vp]),
    "qw_xchg_set_timeout_ms": (None, [_vp, _i32]),
    "qw_op_attn_exchange": (_b, [_vp, _vp, _i32] + [QwRef] * 5 + [_i32] * 8 + [_f32, C.c_int, C.c_int, C.c_int, _i32]),
    "qw_op_attn_exchange_batch": (_b, [_vp, _vp, _i32, _i32] + [_vp] * 8 + [_i32] * 5 + [_f32, C.c_int, C.c_int, C.c_int, _i32]),
    "qw_gpu_last_error": (C.c_char_p, []),
    "qw_gpu_sm_count": (_i32, []),
    "qw_gpu_launch_count": (C.c_uint64, []),
    "qw_gpu_tune": (_b, [C.c_char_p, _i32]),
    "qw_attn_split_plan": (_i32, [_i32, _i32, _vp, _i32, _vp, _vp]),
    "qw_prof_kernels": (None, [_b]),
    "qw_prof_kernel_read": (_b, [C.c_char_p, _vp, _vp, _b]),
    "qw_buf_alloc_device": (_vp, [_sz]),
    "qw_buf_wrap_device": (_vp, [_vp, _sz]),
    "qw_buf_device_ptr": (_vp, [_vp]),
    "qw_buf_upload": (_b, [_vp, _sz, _vp, _sz]),
    "qw_buf_download": (_b, [_vp, _sz, _vp, _sz]),
    "qw_cmd_begin_on_stream": (_vp, [_vp]),
    "qw_op_copy": (None, [_vp, QwRef, QwRef, _sz]),
    "qw_kv_arena_alloc": (_vp, [_i32, _i32, _i32, _i32]),
    "qw_kv_arena_alloc_ex": (_vp, [_i32, _i32, _i32, _i32, C.c_uint32]),
    "qw_kv_read": (_b, [_vp, _i32, _i32, _i32, _i32, _vp, _i32, _i32, _i32]),
    "qw_kv_store": (_b, [_vp, _i32, _i32, _i32, _i32, _vp, _i32, _i32, _i32]),
    "qw_kv_state_bytes": (_sz, [_i32, _i32, _i32, _i32]),
    "qw_kv_element_tag": (C.c_uint32, []),
    "qw_kv_pack": (_b, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _sz]),
    "qw_kv_unpack": (_b, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _sz]),
    "qw_kv_arena_trim": (None, [_vp, _i32]),
    "qw_kv_arena_pages_in_use": (C.c_int64, [_vp]),
    "qw_kv_arena_bytes_committed": (C.c_int64, [_vp]),
    "qw_op_attn_layer_fused": (_b, [_vp] + [QwRef] * 11 + [_i32] * 7 + [_f32, _f32, C.c_int]),
    "qw_op_attn_layer_fused_batch": (_b, [_vp, _i32, _vp, _vp, _vp, _vp, QwRef, QwRef, _vp, QwRef, QwRef, _vp, _vp,
                                          _vp, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _f32, C.c_int]),
    "qw_op_attn_batch": (_b, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32, C.c_int]),
    "qw_op_attn_partial": (_b, [_vp] + [QwRef] * 5 + [_i32] * 8 + [_f32, C.c_int]),
    "qw_op_attn_merge": (None, [_vp] + [QwRef] * 4 + [_i32] * 5 + [C.c_int, C.c_int, C.c_int64]),
    "qw_op_attn_preop": (_b, [_vp] + [QwRef] * 11 + [_i32] * 7 + [_f32, C.c_int, _b]),
    "qw_attn_decode_noalloc": (_b, [_vp] * 5 + [_i32] * 6 + [_f32, C.c_int, _vp, C.c_char_p, _sz]),
    "qw_attn_decode_noalloc_scratch_bytes": (_sz, []),
    "qw_attn_decode_noalloc_status": (_i32, []),
}


def build_library(verbose: bool = False) -> str:
    """Compiles csrc/ for sm_100a with nvcc (works without a GPU)."""
    subprocess.run(["make", "-C", os.path.join(HERE, "csrc"), "all"], check=True,
                   stdout=None if verbose else subprocess.DEVNULL)
    return LIB_PATH


def load_library() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is not built; run `make -C qwasar_b200/csrc` (there is no fallback path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
        fn.restype, fn.argtypes = res, args
    return lib


def ref(buf, off: int = 0) -> QwRef:
    return QwRef(buf, off)


def _ref_array(refs):
    arr = (QwRef * len(refs))(*refs)
    return arr


class Backend:
    """Initialised backend.  Methods carry the reference's op names without the
    qw_ prefix; see include/qwasar_cuda.h for each contract."""

    def __init__(self):
        self.lib = load_library()
        err = C.create_string_buffer(512)
        if not self.lib.qw_gpu_init(err, 512):
            raise RuntimeError("qw_gpu_init failed: " + err.value.decode(errors="replace"))

    # -- device / buffers
    def name(self):
        return self.lib.qw_gpu_name().decode()

    def last_error(self):
        e = self.lib.qw_gpu_last_error()
        return e.decode() if e else None

    def sm_count(self):
        return int(self.lib.qw_gpu_sm_count())

    def launch_count(self):
        return int(self.lib.qw_gpu_launch_count())

    def tune(self, knob, value):
        return bool(self.lib.qw_gpu_tune(knob.encode(), value))

    def prof_kernels(self, on):
        self.lib.qw_prof_kernels(bool(on))

    def prof_kernel_read(self, name, reset=True):
        ms, n = C.c_double(0), C.c_int64(0)
        ok = self.lib.qw_prof_kernel_read(name.encode(), C.addressof(ms), C.addressof(n), reset)
        return (ms.value, n.value) if ok else (0.0, 0)

    def buf_alloc(self, n):
        b = self.lib.qw_buf_alloc(n)
        if not b:
            raise MemoryError(self.last_error())
        return b

    def buf_alloc_device(self, n):
        b = self.lib.qw_buf_alloc_device(n)
        if not b:
            raise MemoryError(self.last_error())
        return b

    def buf_wrap_device(self, ptr, n):
        b = self.lib.qw_buf_wrap_device(ptr, n)
        if not b:
            raise MemoryError("qw_buf_wrap_device failed")
        return b

    def buf_free(self, b):
        self.lib.qw_buf_free(b)

    def buf_contents(self, b):
        return self.lib.qw_buf_contents(b)

    def buf_length(self, b):
        return int(self.lib.qw_buf_length(b))

    def buf_upload(self, b, off, arr):
        if not self.lib.qw_buf_upload(b, off, arr.ctypes.data, arr.nbytes):
            raise RuntimeError(self.last_error())

    def buf_download(self, b, off, arr):
        if not self.lib.qw_buf_download(b, off, arr.ctypes.data, arr.nbytes):
            raise RuntimeError(self.last_error())

    def view(self, b, dtype, count=None, off=0):
        """numpy view of a shared buffer's host side (what qw_buf_contents returns)."""
        import numpy as np
        p = self.buf_contents(b)
        if not p:
            raise ValueError("buffer has no host side")
        n = self.buf_length(b) - off
        raw = (C.c_uint8 * n).from_address(p + off)
        a = np.frombuffer(raw, dtype=dtype)
        return a if count is None else a[:count]

    # -- arena
    def kv_arena_alloc(self, n_layers, kv_heads, max_ctx, head_dim=256, shuffle_seed=0):
        b = self.lib.qw_kv_arena_alloc_ex(n_layers, kv_heads, max_ctx, head_dim, shuffle_seed)
        if not b:
            raise MemoryError(self.last_error())
        return b

    def kv_pool_alloc(self, max_bytes, shuffle_seed=0):
        b = self.lib.qw_kv_pool_alloc(max_bytes, shuffle_seed)
        if not b:
            raise MemoryError(self.last_error())
        return b

    def kv_arena_alloc_in(self, pool, n_layers, kv_heads, max_ctx, head_dim=256):
        b = self.lib.qw_kv_arena_alloc_in(pool, n_layers, kv_heads, max_ctx, head_dim)
        if not b:
            raise MemoryError(self.last_error())
        return b

    # -- the exchange of partials between GPUs
    def xchg_create(self, n_ranks, rank, max_rows_heads):
        x = self.lib.qw_xchg_create(n_ranks, rank, max_rows_heads)
        if not x:
            raise RuntimeError(self.last_error())
        return x

    def xchg_export(self, x) -> bytes:
        h = C.create_string_buffer(int(self.lib.qw_xchg_handle_bytes()))
        if not self.lib.qw_xchg_export(x, h):
            raise RuntimeError(self.last_error())
        return h.raw

    def xchg_attach(self, x, peer_rank, handle: bytes):
        h = C.create_string_buffer(handle, len(handle))
        if not self.lib.qw_xchg_attach(x, peer_rank, h):
            raise RuntimeError(self.last_error())

    def kv_read(self, cache, layer, head, pos0, n, kv_heads, max_ctx, head_dim=256):
        import numpy as np
        out = np.empty((n, head_dim), np.uint16)
        if not self.lib.qw_kv_read(cache, layer, head, pos0, n, out.ctypes.data, kv_heads, max_ctx, head_dim):
            raise RuntimeError(self.last_error())
        return out

    def kv_store(self, cache, layer, head, pos0, rows_u16, kv_heads, max_ctx, head_dim=256):
        import numpy as np
        a = np.ascontiguousarray(rows_u16, np.uint16)
        if not self.lib.qw_kv_store(cache, layer, head, pos0, a.shape[0], a.ctypes.data, kv_heads, max_ctx, head_dim):
            raise RuntimeError(self.last_error())

    def kv_pack(self, kcache, vcache, n_layers, kv_heads, max_ctx, n_tokens, head_dim=256):
        """The KV section of the reference's packed session state as uint16
        [n_layers, kv_heads, 2 (K, V), n_tokens, head_dim]."""
        import numpy as np
        out = np.empty((n_layers, kv_heads, 2, n_tokens, head_dim), np.uint16)
        assert out.nbytes == self.lib.qw_kv_state_bytes(n_layers, kv_heads, head_dim, n_tokens) or n_tokens == 0
        if not self.lib.qw_kv_pack(kcache, vcache, n_layers, kv_heads, max_ctx, head_dim, n_tokens, out.ctypes.data, out.nbytes):
            raise RuntimeError(self.last_error())
        return out

    def kv_unpack(self, kcache, vcache, packed_u16, max_ctx):
        import numpy as np
        a = np.ascontiguousarray(packed_u16, np.uint16)
        n_layers, kv_heads, _, n_tokens, head_dim = a.shape
        if not self.lib.qw_kv_unpack(kcache, vcache, n_layers, kv_heads, max_ctx, head_dim, n_tokens, a.ctypes.data, a.nbytes):
            raise RuntimeError(self.last_error())

    # -- command buffers
    def cmd_begin(self, stream=None):
        c = self.lib.qw_cmd_begin() if stream is None else self.lib.qw_cmd_begin_on_stream(stream)
        if not c:
            raise RuntimeError("qw_cmd_begin failed")
        return c

    def cmd_wait(self, c, check=True):
        self.lib.qw_cmd_wait(c)
        e = self.lib.qw_cmd_error(c)
        if check and e:
            raise RuntimeError("GPU error: " + e.decode(errors="replace"))
        return e.decode() if e else None

    def cmd_free(self, c):
        self.lib.qw_cmd_free(c)

    def cmd_error(self, c):
        e = self.lib.qw_cmd_error(c)
        return e.decode() if e else None

    # -- ops: thin forwards (positional arguments exactly as in the header)
    def __getattr__(self, name):
        if name.startswith("op_") or name in ("rope_tables", "cmd_commit", "cmd_flush", "cmd_parallel", "cmd_mark",
                                               "kv_arena_trim", "kv_arena_pages_in_use", "kv_arena_bytes_committed",
                                               "kv_pool_bytes_committed", "xchg_free", "xchg_attach_local", "xchg_set_timeout_ms",
                                               "gpu_device_count", "gpu_init_multi", "gpu_select", "gpu_current",
                                               "prof_report", "prof_reset"):
            return getattr(self.lib, "qw_" + name)
        raise AttributeError(name)

    def op_attn_layer_fused_batch(self, c, outs, qgs, ks, vs, qw, kw, poss, axis, inv_freq, kcs, vcs, base_pos,
                                  rows, q_heads, kv_heads, head_dim, rotary_dim, max_ctx, eps, scale, io):
        n = len(outs)
        bp = (C.c_int32 * n)(*base_pos)
        arrs = [_ref_array(x) for x in (outs, qgs, ks, vs, poss, kcs, vcs)]
        return self.lib.qw_op_attn_layer_fused_batch(
            c, n, C.addressof(arrs[0]), C.addressof(arrs[1]), C.addressof(arrs[2]), C.addressof(arrs[3]), qw, kw,
            C.addressof(arrs[4]), axis, inv_freq, C.addressof(arrs[5]), C.addressof(arrs[6]), C.addressof(bp),
            rows, q_heads, kv_heads, head_dim, rotary_dim, max_ctx, eps, scale, io)

    def op_attn_exchange_batch(self, c, x, phase, outs, gates, qs, kcs, vcs, base_pos, key_lo, key_hi, rows, q_heads, kv_heads,
                               head_dim, max_ctx, scale, q_dtype, out_dtype, gate_dtype, gate_stride):
        n = len(outs)
        ints = [(C.c_int32 * n)(*v) for v in (base_pos, key_lo, key_hi)]
        arrs = [_ref_array(v) for v in (outs, gates if gates else [NULL_REF] * n, qs, kcs, vcs)]
        return self.lib.qw_op_attn_exchange_batch(
            c, x, phase, n, C.addressof(arrs[0]), C.addressof(arrs[1]) if gates else None, C.addressof(arrs[2]),
            C.addressof(arrs[3]), C.addressof(arrs[4]), C.addressof(ints[0]), C.addressof(ints[1]), C.addressof(ints[2]),
            rows, q_heads, kv_heads, head_dim, max_ctx, scale, q_dtype, out_dtype, gate_dtype, gate_stride)

    def op_attn_batch(self, c, outs, qs, kcs, vcs, base_pos, rows, q_heads, kv_heads, head_dim, max_ctx, scale, io):
        n = len(outs)
        bp = (C.c_int32 * n)(*base_pos)
        arrs = [_ref_array(x) for x in (outs, qs, kcs, vcs)]
        return self.lib.qw_op_attn_batch(c, n, C.addressof(arrs[0]), C.addressof(arrs[1]), C.addressof(arrs[2]),
                                         C.addressof(arrs[3]), C.addressof(bp), rows, q_heads, kv_heads, head_dim,
                                         max_ctx, scale, io)
