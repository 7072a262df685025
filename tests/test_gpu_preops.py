"""Pre/post ops through the C ABI against the oracle -- the checks of the reference's
tests/test_ops.c (norm :64-92, rope :186-261, split :308-333) and the KV-append
memcmp of tests/test_attn.c:128-130."""
import numpy as np
import pytest

from conftest import rel_l2, xorshift_fill
from gpu_util import Bufs, QwRef, NULL_REF
from qwasar_b200 import synth

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_split_heads2_exact(be, oracle):
    rows, heads, dim = 5, 24, 256
    src = xorshift_fill(rows * heads * 2 * dim, 0x4242).reshape(rows, heads, 2 * dim)
    with Bufs(be) as B:
        sb, _ = B.shared(src)
        ab, av = B.shared_empty((rows, heads, dim), np.float32, 7.0)
        bb, bv = B.shared_empty((rows, heads, dim), np.float32, 7.0)
        c = be.cmd_begin()
        be.op_split_heads2(c, QwRef(ab, 0), QwRef(bb, 0), QwRef(sb, 0), rows, heads, dim)
        be.cmd_wait(c); be.cmd_free(c)
        wa, wb = oracle.split_heads2(src, rows, heads, dim)
        assert np.array_equal(bits(av), bits(wa)) and np.array_equal(bits(bv), bits(wb))


@pytest.mark.parametrize("rows,weighted,out_scale", [(24, True, 1.0), (4 * 7, True, 1.0), (6, False, 1.0),
                                                     (33, False, 0.0625)])
def test_rms_norm(be, oracle, rows, weighted, out_scale):
    """q_norm / k_norm shapes: 256-wide rows; max relative error < 1e-5 (tests/test_ops.c:85)."""
    x = xorshift_fill(rows * 256, 0x1234 + rows).reshape(rows, 256)
    w = synth.f32_to_bf16_bits(1.0 + 0.1 * xorshift_fill(256, 0x99)) if weighted else None
    with Bufs(be) as B:
        xb, _ = B.shared(x)
        yb, yv = B.shared_empty((rows, 256), np.float32)
        wref = QwRef(B.shared(w)[0], 0) if weighted else NULL_REF
        c = be.cmd_begin()
        be.op_rms_norm(c, QwRef(yb, 0), QwRef(xb, 0), wref, 256, rows, 1e-6, out_scale)
        be.cmd_wait(c); be.cmd_free(c)
        want = oracle.rms_norm(x, w, 256, rows, 1e-6, out_scale)
        err = np.max(np.abs(yv - want) / np.maximum(np.abs(want), 1e-3 * np.abs(want).max()))
        assert err < 1e-5


@pytest.mark.parametrize("rows,heads,multimodal,base", [(1, 24, False, 0), (8, 24, False, 100), (5, 4, True, 3),
                                                        (3, 4, False, 262000)])
def test_rope_partial(be, oracle, rows, heads, multimodal, base):
    """Text, multimodal and far positions (tests/test_ops.c:397-402): rel-L2 < 1e-6, max abs
    < 1e-5 (a few 1e-6 at position 262000, where cosf/sinf differ in the last bit of a
    2.6e5 rad argument), dims past rotary_dim bitwise untouched, pair norms preserved."""
    hd, rd = 256, 64
    axis, inv = oracle.rope_tables()
    x = xorshift_fill(rows * heads * hd, 0x777).reshape(rows, heads, hd)
    pos = synth.positions(base, rows)
    if multimodal:
        pos[1] = 7 + np.arange(rows); pos[2] = 40 + np.arange(rows)
    with Bufs(be) as B:
        xb, xv = B.shared(x)
        pb, _ = B.shared(pos); ab, _ = B.shared(axis); fb, _ = B.shared(inv)
        c = be.cmd_begin()
        be.op_rope_partial(c, QwRef(xb, 0), QwRef(pb, 0), QwRef(ab, 0), QwRef(fb, 0), rows, heads, hd, rd)
        be.cmd_wait(c); be.cmd_free(c)
        want = oracle.rope_partial(x, pos, axis, inv, rows, heads, hd, rd)
        assert rel_l2(xv, want) < 1e-6
        assert np.abs(xv - want).max() < 1e-5
        assert np.array_equal(bits(xv[..., rd:]), bits(x[..., rd:]))
        n0 = np.sum(x[..., :rd].astype(np.float64) ** 2); n1 = np.sum(xv[..., :rd].astype(np.float64) ** 2)
        assert abs(n0 - n1) / n0 < 1e-5


def test_mul_sigmoid(be, oracle):
    n = 3 * 24 * 256
    y = xorshift_fill(n, 0x31) * 3; g = xorshift_fill(n, 0x32) * 8
    with Bufs(be) as B:
        yb, yv = B.shared(y); gb, _ = B.shared(g)
        c = be.cmd_begin()
        be.op_mul_sigmoid(c, QwRef(yb, 0), QwRef(gb, 0), n)
        be.cmd_wait(c); be.cmd_free(c)
        assert np.abs(yv - oracle.mul_sigmoid(y, g)).max() < 1e-6


@pytest.mark.parametrize("base,rows", [(0, 1), (5, 3), (63, 2), (64, 64), (100, 37)])
def test_kv_write_bit_exact_linear(be, oracle, base, rows):
    """memcmp-equal caches, whole buffer, stale tail included (tests/test_attn.c:89-130)."""
    kvh, hd, ctx = 4, 256, 256
    k = xorshift_fill(rows * kvh * hd, 0x2727).reshape(rows, kvh, hd) * 4
    v = xorshift_fill(rows * kvh * hd, 0x3737).reshape(rows, kvh, hd) * 4
    kc = np.full((kvh, ctx, hd), oracle.to_cache(np.float32([30.0]))[0], np.uint16)
    vc = np.full((kvh, ctx, hd), oracle.to_cache(np.float32([-999.0]))[0], np.uint16)
    with Bufs(be) as B:
        kcb, kcv = B.shared(kc); vcb, vcv = B.shared(vc)
        kb, _ = B.shared(k); vb, _ = B.shared(v)
        c = be.cmd_begin()
        be.op_kv_write(c, QwRef(kcb, 0), QwRef(vcb, 0), QwRef(kb, 0), QwRef(vb, 0), rows, kvh, hd, ctx, base)
        be.cmd_wait(c); be.cmd_free(c)
        oracle.kv_write(kc, vc, k, v, rows, kvh, hd, ctx, base)
        assert np.array_equal(kcv, kc) and np.array_equal(vcv, vc)


def test_kv_write_bit_exact_arena_layers(be, oracle):
    """The same through a paged arena with a permuted page order, at a layer offset the way
    the graph addresses it (kv_stride * fi * 2 bytes, qwasar_graph.c:624,646-649); appends in
    several steps crossing page boundaries; logical contents read back by qw_kv_read."""
    kvh, hd, ctx, layers = 2, 256, 300, 3
    layer_bytes = kvh * ctx * hd * 2
    with Bufs(be) as B:
        ka = B.arena(layers, kvh, ctx, seed=0xBEEF); va = B.arena(layers, kvh, ctx, seed=0xF00D)
        want_k = np.zeros((layers, kvh, ctx, hd), np.uint16); want_v = np.zeros_like(want_k)
        base = {0: 0, 1: 0, 2: 0}
        steps = [(1, 70), (0, 1), (2, 130), (1, 1), (0, 64), (1, 100), (0, 3)]
        for i, (layer, rows) in enumerate(steps):
            k = xorshift_fill(rows * kvh * hd, 0x100 + i).reshape(rows, kvh, hd)
            v = xorshift_fill(rows * kvh * hd, 0x200 + i).reshape(rows, kvh, hd)
            kb, _ = B.shared(k); vb, _ = B.shared(v)
            c = be.cmd_begin()
            be.op_kv_write(c, QwRef(ka, layer * layer_bytes), QwRef(va, layer * layer_bytes), QwRef(kb, 0),
                           QwRef(vb, 0), rows, kvh, hd, ctx, base[layer])
            be.cmd_wait(c); be.cmd_free(c)
            oracle.kv_write(want_k[layer], want_v[layer], k, v, rows, kvh, hd, ctx, base[layer])
            base[layer] += rows
        for layer in range(layers):
            for h in range(kvh):
                got_k = be.kv_read(ka, layer, h, 0, ctx, kvh, ctx)
                got_v = be.kv_read(va, layer, h, 0, ctx, kvh, ctx)
                assert np.array_equal(got_k, want_k[layer, h]) and np.array_equal(got_v, want_v[layer, h])
        pages = sum((base[l] + 63) // 64 for l in range(layers)) * kvh
        assert be.kv_arena_pages_in_use(ka) == pages
        # a rewind gives whole pages back and keeps the rest intact
        be.kv_arena_trim(ka, 64)
        assert be.kv_arena_pages_in_use(ka) == layers * kvh * 1
        assert np.array_equal(be.kv_read(ka, 1, 0, 0, 64, kvh, ctx), want_k[1, 0, :64])


def test_bad_arguments_decline(be):
    """Error convention of the boundary: bool ops return false encoding nothing; positions
    outside the cache surface as a qw_cmd_error string, never as a fault."""
    with Bufs(be) as B:
        qb, _ = B.shared_empty((1, 8, 256), np.float32, 0.0)
        ob, _ = B.shared_empty((1, 8, 256), np.float32, 0.0)
        cb, _ = B.shared_empty((2, 16, 256), np.uint16, 0)
        c = be.cmd_begin()
        r = QwRef
        assert be.op_attn_decode_tensor(c, r(ob, 0), r(qb, 0), r(cb, 0), r(cb, 0), 1, 8, 2, 128, 16, 0, 0.1) is False
        assert be.op_attn_prefill(c, r(ob, 0), r(qb, 0), r(cb, 0), r(cb, 0), 1, 8, 3, 256, 16, 0, 0.1) is False
        assert be.op_attn_decode_split(c, r(ob, 0), r(qb, 0), r(cb, 0), r(cb, 0), 1, 8, 2, 256, 16, 16, 0.1) is False
        assert be.cmd_wait(c, check=False) is None
        be.op_kv_write(c, r(cb, 0), r(cb, 0), r(qb, 0), r(qb, 0), 4, 2, 256, 16, 14)   # rows run past max_ctx
        msg = be.cmd_wait(c, check=False)
        assert msg and "outside the cache" in msg
        be.cmd_free(c)
