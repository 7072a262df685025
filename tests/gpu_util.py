"""Helpers for the GPU parity tests: move numpy arrays through the C ABI the way the
reference's tests do (qw_buf_alloc + qw_buf_contents, tests/test_attn.c:66-76)."""
import numpy as np

from qwasar_b200.backend import QwRef, NULL_REF, F32, BF16  # noqa: F401
from qwasar_b200 import synth


class Bufs:
    """Owns qw_bufs for one test and frees them at exit."""

    def __init__(self, be):
        self.be = be
        self.all = []

    def shared(self, arr):
        """Shared buffer holding a copy of arr; returns (buf, view)."""
        arr = np.ascontiguousarray(arr)
        b = self.be.buf_alloc(max(arr.nbytes, 16))
        self.all.append(b)
        view = self.be.view(b, arr.dtype, arr.size).reshape(arr.shape)
        view[...] = arr
        return b, view

    def shared_empty(self, shape, dtype, fill=None):
        b = self.be.buf_alloc(max(int(np.prod(shape)) * np.dtype(dtype).itemsize, 16))
        self.all.append(b)
        view = self.be.view(b, dtype, int(np.prod(shape))).reshape(shape)
        if fill is not None:
            view[...] = fill
        return b, view

    def device(self, arr):
        arr = np.ascontiguousarray(arr)
        b = self.be.buf_alloc_device(max(arr.nbytes, 16))
        self.all.append(b)
        self.be.buf_upload(b, 0, arr)
        return b

    def arena(self, n_layers, kv_heads, max_ctx, seed=0):
        b = self.be.kv_arena_alloc(n_layers, kv_heads, max_ctx, 256, seed)
        self.all.append(b)
        return b

    def close(self):
        for b in self.all:
            self.be.buf_free(b)
        self.all = []

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def to_io(arr_f32, io):
    """float32 array -> what the ABI reads for that io dtype."""
    return synth.f32_to_bf16_bits(arr_f32) if io == BF16 else np.ascontiguousarray(arr_f32, np.float32)


def from_io(view, io):
    return synth.bf16_bits_to_f32(view) if io == BF16 else np.array(view, np.float32)


def io_np(io):
    return np.uint16 if io == BF16 else np.float32


def arena_fill(be, cache, layer, bits, kv_heads, max_ctx):
    """Stores bits [kv_heads, n, 256] at positions [0, n) of `layer`."""
    for h in range(kv_heads):
        be.kv_store(cache, layer, h, 0, bits[h], kv_heads, max_ctx)


def arena_read(be, cache, layer, n, kv_heads, max_ctx):
    return np.stack([be.kv_read(cache, layer, h, 0, n, kv_heads, max_ctx) for h in range(kv_heads)])
