"""ctypes front end of the CPU oracle (oracle/qw_attn_oracle.c) and of the
reference's own qwasar_cpu.c compiled into oracle/_ref/.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's cpu_baseline / reference arm.  Nothing under qwasar_b200/ imports
this module.

`Oracle` is this repository's restatement; `RefCpu` is the reference source
itself (present when oracle/_ref/ was built in a container that has the
reference checkout; the prebuilt objects then travel with the tree)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BF16, F16 = 0, 1

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i32, _f32, _sz, _int = C.c_int32, C.c_float, C.c_size_t, C.c_int


def build(quiet: bool = True) -> None:
    """Runs oracle/Makefile (restatement always; _ref only where the
    reference checkout exists)."""
    subprocess.run(["make", "-C", HERE, "all"], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _load(path: str) -> C.CDLL:
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} missing: run `make -C oracle`")
    return C.CDLL(path)


def _opt(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Oracle:
    """The restatement.  fast=True loads the -O3 -ffast-math build (timing only)."""

    def __init__(self, fast: bool = False):
        name = "libqworacle_fast.so" if fast else "libqworacle.so"
        path = os.path.join(HERE, "_build", name)
        if not os.path.exists(path):
            build()
        L = self.lib = _load(path)
        L.orc_cache_down_n.argtypes = [_u16p, _f32p, _sz, _int]
        L.orc_cache_up_n.argtypes = [_f32p, _u16p, _sz, _int]
        L.orc_split_heads2.argtypes = [_f32p, _f32p, _f32p, _i32, _i32, _i32]
        L.orc_rms_norm.argtypes = [_f32p, _f32p, C.c_void_p, _i32, _i32, _f32, _f32]
        L.orc_rope_tables.argtypes = [_u8p, _f32p, _i32, _f32, _i32p]
        L.orc_rope_partial.argtypes = [_f32p, _i32p, _u8p, _f32p, _i32, _i32, _i32, _i32]
        L.orc_kv_write.argtypes = [_u16p, _u16p, _f32p, _f32p, _i32, _i32, _i32, _i32, _i32, _int]
        L.orc_attn_decode.argtypes = [_f32p, _f32p, _u16p, _u16p, _i32, _i32, _i32, _i32, _i32,
                                      _i32, _f32, _int, _int]
        L.orc_mul_sigmoid.argtypes = [_f32p, _f32p, _sz]
        L.orc_attn_masked.argtypes = [C.c_void_p] * 5 + [_i32] * 6 + [_f32, _int]
        L.orc_attn_masked.restype = None
        L.orc_qmv_q4.argtypes = [C.c_void_p] * 5 + [_i32] * 4
        L.orc_qmv_q4.restype = None
        L.orc_qsa_scores.argtypes = [C.c_void_p] * 6 + [_i32] * 7 + [_f32]
        L.orc_qsa_scores.restype = None
        L.orc_qsa_select.argtypes = [C.c_void_p] * 3 + [_i32] * 6
        L.orc_qsa_select.restype = None
        L.orc_attn_partial.argtypes = [_f32p, _f32p, _f32p, C.c_void_p, C.c_void_p, _i32, _i32,
                                       _i32, _f32, _int]
        L.orc_attn_merge.argtypes = [_f32p, _f32p, _f32p, _i32, _i32, C.c_void_p]
        L.orc_attn_layer.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_void_p, C.c_void_p, _i32p,
                                     _u8p, _f32p, _u16p, _u16p, _i32, _i32, _i32, _i32, _i32,
                                     _i32, _i32, _f32, _f32, _int, _int, C.c_void_p, C.c_void_p]
        L.orc_max_threads.restype = _int
        self.max_threads = int(L.orc_max_threads())

    # -- conversions
    def to_cache(self, x, fmt=BF16):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self.lib.orc_cache_down_n(out.reshape(-1), x.reshape(-1), x.size, fmt)
        return out

    def from_cache(self, h, fmt=BF16):
        h = np.ascontiguousarray(h, np.uint16)
        out = np.empty(h.shape, np.float32)
        self.lib.orc_cache_up_n(out.reshape(-1), h.reshape(-1), h.size, fmt)
        return out

    # -- ops (same argument meaning as the reference's qw_cpu_* twins)
    def split_heads2(self, src, rows, heads, dim):
        a = np.empty((rows, heads, dim), np.float32)
        b = np.empty((rows, heads, dim), np.float32)
        self.lib.orc_split_heads2(a, b, np.ascontiguousarray(src, np.float32), rows, heads, dim)
        return a, b

    def rms_norm(self, x, w, dim, rows, eps, out_scale=1.0):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.lib.orc_rms_norm(y, x, _opt(w), dim, rows, eps, out_scale)
        return y

    def rope_tables(self, rotary_dim=64, theta=1e7, section=(11, 11, 10)):
        axis = np.zeros(rotary_dim // 2, np.uint8)
        inv = np.zeros(rotary_dim // 2, np.float32)
        self.lib.orc_rope_tables(axis, inv, rotary_dim, theta, np.asarray(section, np.int32))
        return axis, inv

    def rope_partial(self, x, pos, axis, inv_freq, rows, heads, head_dim, rotary_dim):
        x = np.array(x, np.float32, copy=True, order="C")
        self.lib.orc_rope_partial(x, np.ascontiguousarray(pos, np.int32), axis, inv_freq,
                                  rows, heads, head_dim, rotary_dim)
        return x

    def kv_write(self, kc, vc, k, v, rows, kv_heads, head_dim, max_ctx, base_pos, fmt=BF16):
        self.lib.orc_kv_write(kc, vc, np.ascontiguousarray(k, np.float32),
                              np.ascontiguousarray(v, np.float32), rows, kv_heads, head_dim,
                              max_ctx, base_pos, fmt)

    def attn_decode(self, q, kc, vc, rows, q_heads, kv_heads, head_dim, max_ctx, base_pos,
                    scale, fmt=BF16, threads=0):
        q = np.ascontiguousarray(q, np.float32)
        out = np.empty((rows, q_heads, head_dim), np.float32)
        self.lib.orc_attn_decode(out, q, kc, vc, rows, q_heads, kv_heads, head_dim, max_ctx,
                                 base_pos, scale, fmt, threads or self.max_threads)
        return out

    def attn_masked(self, q, kc, vc, lists, rows, q_heads, kv_heads, head_dim, max_ctx, scale, fmt=BF16):
        """lists: uint32 [rows, 1 + cap] (count, then positions ascending)."""
        q = np.ascontiguousarray(q, np.float32)
        lists = np.ascontiguousarray(lists, np.uint32)
        out = np.empty((rows, q_heads, head_dim), np.float32)
        self.lib.orc_attn_masked(out.ctypes.data_as(C.c_void_p), q.ctypes.data_as(C.c_void_p), kc.ctypes.data_as(C.c_void_p),
                                 vc.ctypes.data_as(C.c_void_p), lists.ctypes.data_as(C.c_void_p), C.c_int32(lists.shape[1]),
                                 C.c_int32(rows), C.c_int32(q_heads), C.c_int32(kv_heads), C.c_int32(head_dim),
                                 C.c_int32(max_ctx), C.c_float(scale), C.c_int(fmt))
        return out

    def qmv_q4(self, x, w, scales, biases, k, n, rows, group):
        x = np.ascontiguousarray(x, np.float32); w = np.ascontiguousarray(w, np.uint32)
        sc = np.ascontiguousarray(scales, np.uint16); bi = np.ascontiguousarray(biases, np.uint16)
        y = np.empty((rows, n), np.float32)
        self.lib.orc_qmv_q4(y.ctypes.data, x.ctypes.data, w.ctypes.data, sc.ctypes.data, bi.ctypes.data, k, n, rows, group)
        return y

    def qsa_scores(self, qn, ikeys, k_norm_bits, inv_freq, rows, nq, d, ratio, base_pos, rotary_dim, max_blocks, eps):
        """Returns (scores [rows, max_blocks] with NaN where no block is complete, pool [max_blocks, d])."""
        qn = np.ascontiguousarray(qn, np.float32); ikeys = np.ascontiguousarray(ikeys, np.float32)
        w = np.ascontiguousarray(k_norm_bits, np.uint16); f = np.ascontiguousarray(inv_freq, np.float32)
        scores = np.full((rows, max_blocks), np.nan, np.float32); pool = np.zeros((max_blocks, d), np.float32)
        self.lib.orc_qsa_scores(scores.ctypes.data, pool.ctypes.data, qn.ctypes.data, ikeys.ctypes.data, w.ctypes.data,
                                f.ctypes.data, rows, nq, d, ratio, base_pos, rotary_dim, max_blocks, eps)
        return scores, pool

    def qsa_select(self, scores, rows, ratio, base_pos, block_topk, max_ctx):
        """Returns (mask uint8 [rows, max_ctx] with 255 where not written, list uint32 [rows, 1 + cap])."""
        scores = np.ascontiguousarray(scores, np.float32)
        mask = np.full((rows, max_ctx), 255, np.uint8)
        lists = np.full((rows, 1 + block_topk * ratio + ratio), 0xFFFFFFF0, np.uint32)
        self.lib.orc_qsa_select(mask.ctypes.data, lists.ctypes.data, scores.ctypes.data, rows, ratio, base_pos, block_topk,
                                max_ctx, scores.shape[1])
        return mask, lists

    def mul_sigmoid(self, y, gate):
        y = np.array(y, np.float32, copy=True, order="C")
        self.lib.orc_mul_sigmoid(y.reshape(-1), np.ascontiguousarray(gate, np.float32).reshape(-1),
                                 y.size)
        return y

    def attn_partial(self, q, kh, vh, t0, t1, head_dim, scale, fmt=BF16):
        acc = np.empty(head_dim, np.float32)
        stat = np.empty(2, np.float32)
        self.lib.orc_attn_partial(acc, stat, np.ascontiguousarray(q, np.float32),
                                  kh.ctypes.data_as(C.c_void_p), vh.ctypes.data_as(C.c_void_p),
                                  t0, t1, head_dim, scale, fmt)
        return acc, stat

    def attn_merge(self, pacc, pstat, gate=None):
        pacc = np.ascontiguousarray(pacc, np.float32)
        pstat = np.ascontiguousarray(pstat, np.float32)
        parts, hd = pacc.shape
        out = np.empty(hd, np.float32)
        g = None if gate is None else np.ascontiguousarray(gate, np.float32)
        self.lib.orc_attn_merge(out, pacc, pstat, parts, hd, _opt(g))
        return out

    def attn_layer(self, qg, k, v, qw, kw, pos, axis, inv_freq, kc, vc, rows, q_heads, kv_heads,
                   head_dim, rotary_dim, max_ctx, base_pos, eps, scale, fmt=BF16, threads=0,
                   want_post=False):
        out = np.empty((rows, q_heads, head_dim), np.float32)
        qp = np.empty((rows, q_heads, head_dim), np.float32) if want_post else None
        kp = np.empty((rows, kv_heads, head_dim), np.float32) if want_post else None
        self.lib.orc_attn_layer(out, np.ascontiguousarray(qg, np.float32),
                                np.ascontiguousarray(k, np.float32),
                                np.ascontiguousarray(v, np.float32), _opt(qw), _opt(kw),
                                np.ascontiguousarray(pos, np.int32), axis, inv_freq, kc, vc,
                                rows, q_heads, kv_heads, head_dim, rotary_dim, max_ctx, base_pos,
                                eps, scale, fmt, threads or self.max_threads, _opt(qp), _opt(kp))
        return (out, qp, kp) if want_post else out


class RefCpu:
    """The reference's unmodified qwasar_cpu.c, compiled by oracle/Makefile.
    kind: 'bf16' (this build's cache type), 'f16' (the shipped one), 'bf16_fast'
    (the reference's own -O3 -ffast-math flags; timing only)."""

    def __init__(self, kind: str = "bf16"):
        L = self.lib = _load(os.path.join(HERE, "_ref", f"libqwcpu_{kind}.so"))
        L.qw_f32_to_f16_c.argtypes = [_f32]
        L.qw_f32_to_f16_c.restype = C.c_uint16
        L.qw_f16_to_f32_c.argtypes = [C.c_uint16]
        L.qw_f16_to_f32_c.restype = _f32
        L.qw_cpu_rms_norm.argtypes = [_f32p, _f32p, C.c_void_p, _i32, _i32, _f32, _f32]
        L.qw_rope_tables.argtypes = [_u8p, _f32p, _i32, _f32, _i32p]
        L.qw_cpu_rope_partial.argtypes = [_f32p, _i32p, _u8p, _f32p, _i32, _i32, _i32, _i32]
        L.qw_cpu_kv_write.argtypes = [_u16p, _u16p, _f32p, _f32p, _i32, _i32, _i32, _i32, _i32]
        L.qw_cpu_attn_decode.argtypes = [_f32p, _f32p, _u16p, _u16p, _i32, _i32, _i32, _i32,
                                         _i32, _i32, _f32]
        L.qwref_attn_decode_mt.argtypes = [_f32p, _f32p, _u16p, _u16p, _i32, _i32, _i32, _i32,
                                           _i32, _i32, _f32, _int]
        L.qwref_max_threads.restype = _int
        self.max_threads = int(L.qwref_max_threads())

    @staticmethod
    def available(kind: str = "bf16") -> bool:
        return os.path.exists(os.path.join(HERE, "_ref", f"libqwcpu_{kind}.so"))

    def to_cache_scalar(self, v: float) -> int:
        return int(self.lib.qw_f32_to_f16_c(v))

    def rms_norm(self, x, w, dim, rows, eps, out_scale=1.0):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.lib.qw_cpu_rms_norm(y, x, _opt(w), dim, rows, eps, out_scale)
        return y

    def rope_tables(self, rotary_dim=64, theta=1e7, section=(11, 11, 10)):
        axis = np.zeros(rotary_dim // 2, np.uint8)
        inv = np.zeros(rotary_dim // 2, np.float32)
        self.lib.qw_rope_tables(axis, inv, rotary_dim, theta, np.asarray(section, np.int32))
        return axis, inv

    def rope_partial(self, x, pos, axis, inv_freq, rows, heads, head_dim, rotary_dim):
        x = np.array(x, np.float32, copy=True, order="C")
        self.lib.qw_cpu_rope_partial(x, np.ascontiguousarray(pos, np.int32), axis, inv_freq,
                                     rows, heads, head_dim, rotary_dim)
        return x

    def kv_write(self, kc, vc, k, v, rows, kv_heads, head_dim, max_ctx, base_pos):
        self.lib.qw_cpu_kv_write(kc, vc, np.ascontiguousarray(k, np.float32),
                                 np.ascontiguousarray(v, np.float32), rows, kv_heads, head_dim,
                                 max_ctx, base_pos)

    def attn_decode(self, q, kc, vc, rows, q_heads, kv_heads, head_dim, max_ctx, base_pos,
                    scale, threads=1):
        q = np.ascontiguousarray(q, np.float32)
        out = np.empty((rows, q_heads, head_dim), np.float32)
        if threads == 1:
            self.lib.qw_cpu_attn_decode(out, q, kc, vc, rows, q_heads, kv_heads, head_dim,
                                        max_ctx, base_pos, scale)
        else:
            self.lib.qwref_attn_decode_mt(out, q, kc, vc, rows, q_heads, kv_heads, head_dim,
                                          max_ctx, base_pos, scale, threads or self.max_threads)
        return out

    def qmv_q4(self, x, w, scales, biases, k, n, rows, group):
        """The reference's own qw_cpu_qmv_q4 (qwasar_cpu.c:36-63)."""
        x = np.ascontiguousarray(x, np.float32); w = np.ascontiguousarray(w, np.uint32)
        sc = np.ascontiguousarray(scales, np.uint16); bi = np.ascontiguousarray(biases, np.uint16)
        y = np.empty((rows, n), np.float32)
        fn = self.lib.qw_cpu_qmv_q4
        fn.argtypes = [C.c_void_p] * 5 + [C.c_int32] * 4
        fn.restype = None
        fn(y.ctypes.data, x.ctypes.data, w.ctypes.data, sc.ctypes.data, bi.ctypes.data, k, n, rows, group)
        return y

    def attn_layer(self, qg, k, v, qw, kw, pos, axis, inv_freq, kc, vc, rows, q_heads, kv_heads,
                   head_dim, rotary_dim, max_ctx, base_pos, eps, scale, threads=0):
        """The node composed from the reference's functions in the graph's
        order (qwasar_graph.c:630-659) up to, not including, the output gate:
        the reference has no CPU twin of qw_mul_sigmoid (only the Metal kernel,
        metal/act.metal:29-37), so the caller applies Oracle.mul_sigmoid.
        Returns (pre-gate out, gate, q after norm+rope, k after norm+rope)."""
        qg = np.ascontiguousarray(qg, np.float32).reshape(rows, q_heads, 2 * head_dim)
        q = np.ascontiguousarray(qg[:, :, :head_dim])
        gate = np.ascontiguousarray(qg[:, :, head_dim:])
        q = self.rms_norm(q, qw, head_dim, rows * q_heads, eps)
        kk = self.rms_norm(k, kw, head_dim, rows * kv_heads, eps)
        q = self.rope_partial(q, pos, axis, inv_freq, rows, q_heads, head_dim, rotary_dim)
        kk = self.rope_partial(kk, pos, axis, inv_freq, rows, kv_heads, head_dim, rotary_dim)
        self.kv_write(kc, vc, kk, v, rows, kv_heads, head_dim, max_ctx, base_pos)
        out = self.attn_decode(q, kc, vc, rows, q_heads, kv_heads, head_dim, max_ctx, base_pos,
                               scale, threads=threads or self.max_threads)
        return out, gate, q, kk


class RefFlash:
    """One synthetic attention layer run by the reference's own qwasar_flash_cpu.c
    (oracle/_ref/libqwflashcpu.so, built by oracle/Makefile around ref_flash_driver.c): its block
    selection `qsa_select` (qwasar_flash_cpu.c:346-418) and its composed gated-attention layer
    `qsa_step` (:422-488), fed through 4-bit affine projections as in a bound engine."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(os.path.join(HERE, "_ref", "libqwflashcpu.so"))

    def __init__(self, *, hidden, hidden_out, q_heads, kv_heads, head_dim, idx_heads, idx_dim, budget, ratio, max_ctx,
                 proj, norms, rotary_dim=64, theta=1e7, section=(11, 11, 10), eps=1e-6, group=64):
        """proj: dict name -> (weight uint32 [out, in/8], scales uint16 [out, in/group], biases uint16) for
        q_proj, k_proj, v_proj, o_proj, qk_proj; norms: dict name -> uint16 [dim] or None for q_norm, k_norm,
        idx_q_norm, idx_k_norm."""
        L = self.lib = _load(os.path.join(HERE, "_ref", "libqwflashcpu.so"))
        self.keep = []
        ptrs = []
        for name in ("q_proj", "k_proj", "v_proj", "o_proj", "qk_proj"):
            for a, dt in zip(proj[name], (np.uint32, np.uint16, np.uint16)):
                a = np.ascontiguousarray(a, dt); self.keep.append(a); ptrs.append(a.ctypes.data)
        nptrs = []
        for name in ("q_norm", "k_norm", "idx_q_norm", "idx_k_norm"):
            a = norms.get(name)
            if a is None:
                nptrs.append(None)
            else:
                a = np.ascontiguousarray(a, np.uint16); self.keep.append(a); nptrs.append(a.ctypes.data)
        P = (C.c_void_p * 15)(*ptrs); N = (C.c_void_p * 4)(*nptrs)
        sec = np.asarray(section, np.int32)
        L.qwflash_new.restype = C.c_void_p
        L.qwflash_new.argtypes = [C.c_int] * 6 + [C.c_float, C.c_void_p] + [C.c_int] * 4 + [C.c_float, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        self.h = L.qwflash_new(hidden, hidden_out, q_heads, kv_heads, head_dim, rotary_dim, theta, sec.ctypes.data, idx_heads, idx_dim,
                               budget, ratio, eps, max_ctx, group, P, N)
        L.qwflash_free.argtypes = [C.c_void_p]
        L.qwflash_select.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        L.qwflash_step.argtypes = [C.c_void_p, C.c_void_p, C.c_int] + [C.c_void_p] * 4
        self.dims = dict(hidden=hidden, hidden_out=hidden_out, q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim,
                         idx_heads=idx_heads, idx_dim=idx_dim)

    def select(self, x, pos):
        """(allowed uint8 [pos + 1], qk f32 [(idx_heads + 1) * idx_dim]) for the token at pos; feed positions in order."""
        d = self.dims
        x = np.ascontiguousarray(x, np.float32)
        allowed = np.zeros(pos + 1, np.uint8); qk = np.zeros((d["idx_heads"] + 1) * d["idx_dim"], np.float32)
        self.lib.qwflash_select(self.h, x.ctypes.data, pos, allowed.ctypes.data, qk.ctypes.data)
        return allowed, qk

    def step(self, x, pos):
        """(out [hidden_out], qg [q_heads, 2 * head_dim], k, v [kv_heads, head_dim]) for the token at pos, in order."""
        d = self.dims
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(d["hidden_out"], np.float32); qg = np.zeros((d["q_heads"], 2 * d["head_dim"]), np.float32)
        k = np.zeros((d["kv_heads"], d["head_dim"]), np.float32); v = np.zeros_like(k)
        self.lib.qwflash_step(self.h, x.ctypes.data, pos, out.ctypes.data, qg.ctypes.data, k.ctypes.data, v.ctypes.data)
        return out, qg, k, v

    def close(self):
        if self.h:
            self.lib.qwflash_free(self.h); self.h = None
