"""qw_attn_decode_noalloc: the decode entry point for embedders that must not allocate.

Some hosts of this library own all device memory themselves, or run their decode loop
where a cudaMalloc (which stalls the whole device) is not acceptable.  For them the
library offers one attention call whose scratch is a fixed array inside the library image
instead of a pool that grows on demand.  This test drives it through the C ABI with raw
device pointers and holds its output to the regular entry point's (qw_op_attn_decode_tensor,
the same kernel fed from pooled scratch) on two calls in a row with different inputs, so a
second call is seen to be unaffected by what the first left in the shared array.

The file name sorts after every other test file on purpose: a run that stops at the first
failure has then already executed all the other tests."""
import ctypes as C

import numpy as np
import pytest

from conftest import max_rel_err, rel_l2
from gpu_util import Bufs, QwRef, F32, BF16
from qwasar_b200 import synth

pytestmark = pytest.mark.gpu


def both_ways(be, B, q, kc, vc, rows, qh, kvh, ctx, base, use_stream=False):
    """(existing entry point's output, new entry point's output) for one decode step."""
    qb = B.device(q)
    kcb = B.device(kc); vcb = B.device(vc)
    o_old = B.device(np.full((rows, qh, 256), 7.0, np.float32))
    o_new = B.device(np.full((rows, qh, 256), -7.0, np.float32))
    c = be.cmd_begin()
    assert be.op_attn_decode_tensor(c, QwRef(o_old, 0), QwRef(qb, 0), QwRef(kcb, 0), QwRef(vcb, 0), rows, qh, kvh, 256,
                                    ctx, base, synth.SCALE)
    be.cmd_wait(c); be.cmd_free(c)
    err = C.create_string_buffer(256)
    dp = be.lib.qw_buf_device_ptr
    import torch
    stream = torch.cuda.Stream() if use_stream else None
    ok = be.lib.qw_attn_decode_noalloc(dp(o_new), dp(qb), None, dp(kcb), dp(vcb), rows, qh, kvh, 256, ctx, base,
                                       synth.SCALE, F32, stream.cuda_stream if stream else None, err, 256)
    assert ok, err.value.decode()
    torch.cuda.synchronize()
    assert be.lib.qw_attn_decode_noalloc_status() == 0          # no kernel gave up on a wait
    a = np.empty((rows, qh, 256), np.float32); b = np.empty_like(a)
    be.buf_download(o_old, 0, a); be.buf_download(o_new, 0, b)
    return a, b


def test_noalloc_matches_pooled_entry_point_twice(be, oracle):
    assert be.lib.qw_attn_decode_noalloc_scratch_bytes() == 4 << 20
    rng = np.random.default_rng(2024)
    with Bufs(be) as B:
        # first call: one token deep in a 27B-shaped cache; second call: other depth, grouping and rows
        # (the second on a stream of the caller's instead of the default stream)
        for call, (rows, qh, kvh, base) in enumerate(((1, 24, 4, 5000), (2, 16, 2, 777))):
            ctx = base + rows + 5
            q = synth.normal_bf16(rng, (rows, qh, 256))
            kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
            old, new = both_ways(be, B, q, kc, vc, rows, qh, kvh, ctx, base, use_stream=call == 1)
            assert np.isfinite(new).all()
            assert max_rel_err(new, old) <= 1e-2 and rel_l2(new, old) < 5e-3
            want = oracle.attn_decode(q, kc, vc, rows, qh, kvh, 256, ctx, base, synth.SCALE)
            assert max_rel_err(new, want) <= 1e-2


def test_noalloc_gate_and_bf16(be, oracle):
    """bf16 activations with the sigmoid gate folded in, against the oracle."""
    rng = np.random.default_rng(7)
    rows, qh, kvh, base = 1, 16, 4, 3000
    ctx = base + 8
    q = synth.normal_bf16(rng, (rows, qh, 256)); gate = synth.normal_bf16(rng, (rows, qh, 256))
    kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
    with Bufs(be) as B:
        qb = B.device(synth.f32_to_bf16_bits(q)); gb = B.device(synth.f32_to_bf16_bits(gate))
        kcb = B.device(kc); vcb = B.device(vc)
        ob = B.device(np.zeros((rows, qh, 256), np.uint16))
        err = C.create_string_buffer(256)
        dp = be.lib.qw_buf_device_ptr
        assert be.lib.qw_attn_decode_noalloc(dp(ob), dp(qb), dp(gb), dp(kcb), dp(vcb), rows, qh, kvh, 256, ctx, base,
                                             synth.SCALE, BF16, None, err, 256), err.value.decode()
        import torch
        torch.cuda.synchronize()
        got = np.empty((rows, qh, 256), np.uint16); be.buf_download(ob, 0, got)
    want = oracle.mul_sigmoid(oracle.attn_decode(q, kc, vc, rows, qh, kvh, 256, ctx, base, synth.SCALE), gate)
    assert max_rel_err(synth.bf16_bits_to_f32(got), want) <= 1e-2


def test_noalloc_rejects_what_does_not_fit(be):
    """Shapes past the entry point's limits are refused with a reason; nothing is launched."""
    with Bufs(be) as B:
        buf = B.device(np.zeros(1 << 20, np.uint8))
        p = be.lib.qw_buf_device_ptr(buf)
        err = C.create_string_buffer(256)
        # 8 rows x grouping 6 = 48 query rows per kv head: beyond the 16 this entry point takes
        assert not be.lib.qw_attn_decode_noalloc(p, p, None, p, p, 8, 24, 4, 256, 64, 0, 0.0625, F32, None, err, 256)
        assert b"exceeds 16" in err.value
        assert not be.lib.qw_attn_decode_noalloc(p, p, None, p, p, 1, 24, 4, 128, 64, 0, 0.0625, F32, None, err, 256)
        assert b"head_dim" in err.value
        assert not be.lib.qw_attn_decode_noalloc(p, p, None, p, p, 1, 24, 4, 256, 64, 64, 0.0625, F32, None, err, 256)
        assert b"outside the cache" in err.value
        # 128 kv heads: one partial slot per (SM or kv head) x 16 rows of 1032 bytes no longer fits the 4 MiB
        assert not be.lib.qw_attn_decode_noalloc(p, p, None, p, p, 1, 128, 128, 256, 64, 0, 0.0625, F32, None, err, 256)
        assert b"bytes of scratch" in err.value
