"""Attention kernels through the reference's op signatures, on the shape list and the
three direct property checks of the reference's tests/test_attn.c.

Tolerances.  The per-query kernel is fp32 throughout and is held to the reference's own
bound for its float kernels (rel-L2 < 2e-5, tests/test_attn.c:135-138).  The split-KV and
tiled kernels feed bf16 tensor-core operands (q and the softmax weights are rounded to
bf16, accumulation is fp32): max relative error <= 1e-2 per output vector (see
conftest.max_rel_err) and rel-L2 < 5e-3; the reference allows its own half-staged form
5e-4 with IEEE half's three extra mantissa bits."""
import numpy as np
import pytest

from conftest import max_rel_err, rel_l2, xorshift_fill
from gpu_util import Bufs, QwRef
from qwasar_b200 import synth

pytestmark = pytest.mark.gpu

MAX_CTX = 2048
PER_QUERY, TILED, SPLIT, SPLIT_TENSOR, DISPATCH = "per_query", "tiled", "split", "split_tensor", "qw_op_attn"


def encode(be, c, kind, o, q, kc, vc, rows, qh, kvh, ctx, base, scale):
    a = (c, o, q, kc, vc, rows, qh, kvh, 256, ctx, base, scale)
    if kind == PER_QUERY:
        be.op_attn_decode(*a)
    elif kind == TILED:
        assert be.op_attn_prefill_as(c, True, *a[1:]), "the tiled kernel declined"
    elif kind == SPLIT:
        assert be.op_attn_decode_split(*a), "the split kernel declined"
    elif kind == SPLIT_TENSOR:
        assert be.op_attn_decode_tensor(*a), "the tensor split kernel declined"
    else:
        be.op_attn(*a)


def run_case(be, oracle, kind, base, rows, qh=24, kvh=4, ctx=MAX_CTX):
    """test_attention of tests/test_attn.c:56-141: history through kv_write, every slot past
    base+rows poisoned (K=30, V=-999), kv_write + attention in one command buffer."""
    hd, scale = 256, 0.0625
    kc = np.zeros((kvh, ctx, hd), np.uint16); vc = np.zeros((kvh, ctx, hd), np.uint16)
    if base:
        hk = xorshift_fill(base * kvh * hd, 0x5150).reshape(base, kvh, hd)
        hv = xorshift_fill(base * kvh * hd, 0x6161).reshape(base, kvh, hd)
        oracle.kv_write(kc, vc, hk, hv, base, kvh, hd, ctx, 0)
    kc[:, base + rows:] = oracle.to_cache(np.float32([30.0]))[0]
    vc[:, base + rows:] = oracle.to_cache(np.float32([-999.0]))[0]
    q = xorshift_fill(rows * qh * hd, 0x1717).reshape(rows, qh, hd) * 4   # score spread of a normed query
    k = xorshift_fill(rows * kvh * hd, 0x2727).reshape(rows, kvh, hd)
    v = xorshift_fill(rows * kvh * hd, 0x3737).reshape(rows, kvh, hd)
    with Bufs(be) as B:
        qb, _ = B.shared(q); kb, _ = B.shared(k); vb, _ = B.shared(v)
        ob, ov = B.shared_empty((rows, qh, hd), np.float32)
        ov.view(np.uint32)[...] = 0xCDCDCDCD
        kcb, kcv = B.shared(kc); vcb, vcv = B.shared(vc)
        c = be.cmd_begin()
        r = QwRef
        be.op_kv_write(c, r(kcb, 0), r(vcb, 0), r(kb, 0), r(vb, 0), rows, kvh, hd, ctx, base)
        encode(be, c, kind, r(ob, 0), r(qb, 0), r(kcb, 0), r(vcb, 0), rows, qh, kvh, ctx, base, scale)
        be.cmd_wait(c); be.cmd_free(c)
        oracle.kv_write(kc, vc, k, v, rows, kvh, hd, ctx, base)
        assert np.array_equal(kcv, kc), "kv_write: K cache mismatch"
        assert np.array_equal(vcv, vc), "kv_write: V cache mismatch"
        want = oracle.attn_decode(q, kc, vc, rows, qh, kvh, hd, ctx, base, scale)
        got = np.array(ov)
    assert np.isfinite(got).all()
    return got, want


@pytest.mark.parametrize("base,rows", [(0, 1), (1, 1), (31, 1), (32, 1), (200, 1), (0, 8), (50, 4)])
def test_per_query(be, oracle, base, rows):
    got, want = run_case(be, oracle, PER_QUERY, base, rows)
    assert rel_l2(got, want) < 2e-5


@pytest.mark.parametrize("base,rows", [(0, 16), (0, 32), (0, 37), (5, 64), (300, 100), (1500, 256)])
def test_tiled(be, oracle, base, rows):
    got, want = run_case(be, oracle, TILED, base, rows)
    assert max_rel_err(got, want) <= 1e-2 and rel_l2(got, want) < 5e-3


@pytest.mark.parametrize("kind", [SPLIT, SPLIT_TENSOR])
@pytest.mark.parametrize("base,rows", [(0, 1), (40, 1), (255, 1), (256, 1), (2000, 1), (1990, 5), (1000, 8)])
def test_split(be, oracle, kind, base, rows):
    got, want = run_case(be, oracle, kind, base, rows)
    assert max_rel_err(got, want) <= 1e-2 and rel_l2(got, want) < 5e-3


@pytest.mark.parametrize("kind", [SPLIT_TENSOR, DISPATCH])
@pytest.mark.parametrize("base,rows", [(500, 6), (1200, 9)])
def test_verify_rows_of_a_12_to_1_grouping(be, oracle, kind, base, rows):
    """A Flash-Next-shaped verify block (24 query / 2 KV heads): 6 to 9 rows x 12 heads exceed one
    64-row tile, so the split-KV kernel takes the rows in chunks instead of declining."""
    got, want = run_case(be, oracle, kind, base, rows, qh=24, kvh=2, ctx=1536)
    assert max_rel_err(got, want) <= 1e-2 and rel_l2(got, want) < 5e-3


@pytest.mark.parametrize("qh,kvh", [(16, 4), (16, 2), (24, 2), (8, 8)])
@pytest.mark.parametrize("base,rows", [(0, 1), (97, 1), (700, 3), (10, 20)])
def test_dispatch_other_groupings(be, oracle, qh, kvh, base, rows):
    """qw_op_attn's shape rule over the groupings of the three checkpoints (4:1, 8:1, 12:1)
    and no grouping at all -- the reference's split kernel only takes 6:1."""
    got, want = run_case(be, oracle, DISPATCH, base, rows, qh=qh, kvh=kvh, ctx=1024)
    assert max_rel_err(got, want) <= 1e-2 and rel_l2(got, want) < 5e-3


@pytest.mark.parametrize("kind", [PER_QUERY, SPLIT_TENSOR, DISPATCH])
def test_causality(be, oracle, kind):
    """tests/test_attn.c:148-194: the output is bitwise the same after everything past the
    query's position is overwritten with huge keys."""
    qh, kvh, hd, base, ctx = 24, 4, 256, 40, MAX_CTX
    q = xorshift_fill(qh * hd, 0x8888).reshape(1, qh, hd)
    hk = xorshift_fill((base + 1) * kvh * hd, 0x9999).reshape(base + 1, kvh, hd)
    hv = xorshift_fill((base + 1) * kvh * hd, 0xAAAA).reshape(base + 1, kvh, hd)
    kc = np.zeros((kvh, ctx, hd), np.uint16); vc = np.zeros((kvh, ctx, hd), np.uint16)
    oracle.kv_write(kc, vc, hk, hv, base + 1, kvh, hd, ctx, 0)
    with Bufs(be) as B:
        qb, _ = B.shared(q)
        o1, v1 = B.shared_empty((1, qh, hd), np.float32); o2, v2 = B.shared_empty((1, qh, hd), np.float32)
        kcb, kcv = B.shared(kc); vcb, vcv = B.shared(vc)
        r = QwRef
        c = be.cmd_begin()
        encode(be, c, kind, r(o1, 0), r(qb, 0), r(kcb, 0), r(vcb, 0), 1, qh, kvh, ctx, base, 0.0625)
        be.cmd_wait(c); be.cmd_free(c)
        kcv[:, base + 1:] = oracle.to_cache(np.float32([50.0]))[0]
        vcv[:, base + 1:] = oracle.to_cache(np.float32([-999.0]))[0]
        c = be.cmd_begin()
        encode(be, c, kind, r(o2, 0), r(qb, 0), r(kcb, 0), r(vcb, 0), 1, qh, kvh, ctx, base, 0.0625)
        be.cmd_wait(c); be.cmd_free(c)
        assert np.array_equal(v1.view(np.uint32), v2.view(np.uint32)), "attention read past its own position"


@pytest.mark.parametrize("kind", [PER_QUERY, SPLIT_TENSOR])
@pytest.mark.parametrize("qh,kvh", [(24, 4), (16, 2)])
def test_gqa_and_normalisation(be, oracle, kind, qh, kvh):
    """tests/test_attn.c:199-238: V constant per kv head, so the output names the kv head each
    query head read (h / gqa + 1) and shows the weights sum to one; small integers are exact
    in bf16, so the tensor-op kernel is held to the same 1e-4... loosened to 1e-2 relative of
    the weights' bf16 rounding for it."""
    hd, n, ctx = 256, 33, MAX_CTX
    q = xorshift_fill(qh * hd, 0xBEAD).reshape(1, qh, hd)
    kc = np.zeros((kvh, ctx, hd), np.uint16); vc = np.zeros((kvh, ctx, hd), np.uint16)
    for h in range(kvh):
        vc[h, :n] = oracle.to_cache(np.float32([h + 1.0]))[0]
    with Bufs(be) as B:
        qb, _ = B.shared(q); ob, ov = B.shared_empty((1, qh, hd), np.float32)
        kcb, _ = B.shared(kc); vcb, _ = B.shared(vc)
        c = be.cmd_begin()
        encode(be, c, kind, QwRef(ob, 0), QwRef(qb, 0), QwRef(kcb, 0), QwRef(vcb, 0), 1, qh, kvh, ctx, n - 1, 0.0625)
        be.cmd_wait(c); be.cmd_free(c)
        want = (np.arange(qh) // (qh // kvh) + 1).astype(np.float32)
        dev = np.abs(ov[0] - want[:, None]).max()
        assert dev < (1e-4 if kind == PER_QUERY else 1e-2)


@pytest.mark.parametrize("kind,rows,base", [(TILED, 70, 30), (TILED, 200, 0), (SPLIT_TENSOR, 3, 97), (PER_QUERY, 2, 50)])
def test_tail_of_a_caller_owned_cache_may_hold_anything(be, oracle, kind, rows, base):
    """Cache rows past the last query position never matter (tests/test_attn.c:148-194), even when
    they hold NaN or infinity bit patterns -- a caller-owned buffer promises nothing about them."""
    qh, kvh, ctx, hd = 16, 4, 512, 256
    rng = np.random.default_rng(rows)
    n = base + rows
    kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
    kc[:, n:] = 0x7FC0; vc[:, n:] = 0x7FC0                       # quiet NaN
    kc[:, n + 1::2] = 0x7F80; vc[:, n + 1::2] = 0xFF80           # +inf / -inf
    q = synth.normal_bf16(rng, (rows, qh, hd))
    with Bufs(be) as B:
        qb, _ = B.shared(q)
        ob, ov = B.shared_empty((rows, qh, hd), np.float32)
        kcb = B.device(kc); vcb = B.device(vc)
        c = be.cmd_begin()
        encode(be, c, kind, QwRef(ob, 0), QwRef(qb, 0), QwRef(kcb, 0), QwRef(vcb, 0), rows, qh, kvh, ctx, base, 0.0625)
        be.cmd_wait(c); be.cmd_free(c)
        got = np.array(ov)
    assert np.isfinite(got).all(), "a NaN from beyond the last key reached the output"
    kc[:, n:] = 0; vc[:, n:] = 0
    want = oracle.attn_decode(q, kc, vc, rows, qh, kvh, hd, ctx, base, 0.0625)
    assert max_rel_err(got, want) <= 1e-2


def test_copy_reads_what_an_earlier_op_wrote(be):
    """qw_op_copy inside a command buffer sees the output of the op encoded before it (ops run in
    encoding order and each sees everything before it, qwasar_gpu.h:63-65)."""
    x = np.linspace(-3, 3, 1024).astype(np.float32)
    g = np.ones(1024, np.float32) * 0.5
    with Bufs(be) as B:
        yb, yv = B.shared(x.copy()); gb, _ = B.shared(g)
        db, dv = B.shared_empty((1024,), np.float32, fill=0.0)
        c = be.cmd_begin()
        be.op_mul_sigmoid(c, QwRef(yb, 0), QwRef(gb, 0), 1024)
        be.op_copy(c, QwRef(db, 0), QwRef(yb, 0), 4096)
        be.cmd_wait(c); be.cmd_free(c)
        want = x * (1.0 / (1.0 + np.exp(-0.5)))
        assert np.allclose(np.array(dv), want, rtol=1e-6)
        assert np.array_equal(np.array(dv), np.array(yv))


def test_flush_starts_the_copy_back_and_later_writes_still_arrive(be):
    """qw_cmd_flush (the reference flushes between layers, qwasar_flash_graph.c:657) lets what was written so far
    start its way back to the host; a range that a later op of the same command buffer writes again, and a buffer
    first written after the flush, must still hold their final values after qw_cmd_wait."""
    x = np.linspace(-2, 2, 4096).astype(np.float32)
    g = np.full(4096, 0.25, np.float32)
    sg = 1.0 / (1.0 + np.exp(-0.25))
    with Bufs(be) as B:
        ab, av = B.shared(x.copy()); bb, bv = B.shared(x.copy()); gb, _ = B.shared(g)
        c = be.cmd_begin()
        be.op_mul_sigmoid(c, QwRef(ab, 0), QwRef(gb, 0), 4096)          # a *= s
        be.cmd_flush(c)
        be.op_mul_sigmoid(c, QwRef(ab, 0), QwRef(gb, 0), 4096)          # a *= s again, after its first copy-back began
        be.op_mul_sigmoid(c, QwRef(bb, 0), QwRef(gb, 0), 4096)          # b first written after the flush
        be.cmd_flush(c)
        be.cmd_flush(c)                                                 # nothing new: a no-op
        be.cmd_wait(c); be.cmd_free(c)
        assert np.allclose(np.array(av), x * sg * sg, rtol=2e-6)
        assert np.allclose(np.array(bv), x * sg, rtol=2e-6)
