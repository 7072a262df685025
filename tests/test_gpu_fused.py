"""The fused node (qw_op_attn_layer_fused and its batched form) against the oracle's
composition of the reference functions (qwasar_graph.c:630-659), over plain and paged
caches, fp32 and bf16 activations, and against the committed golden fixtures.

KV append through the fused path: K is normed and roped on the device before its one
rounding to bf16.  The device keeps the CPU code's order for the key rows' sum of squares
(left to right) and takes cos / sin correctly rounded, so every appended K element equals the
oracle's bit for bit, like V (which is only rounded).  The gate on the append op alone is
test_gpu_preops.test_kv_write_bit_exact_*."""
import os
import sys

import numpy as np
import pytest

from conftest import max_rel_err, rel_l2
from gpu_util import Bufs, QwRef, NULL_REF, F32, BF16, to_io, from_io, io_np, arena_fill, arena_read
from oracle.oracle import BF16 as ORC_BF16
from qwasar_b200 import synth

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "attn_golden.npz"))


def check_k_rows(got_bits, want_bits):
    """Appended K: bit-exact against the oracle (the north star's bar for KV append)."""
    differ = got_bits != want_bits
    if differ.any():
        got = synth.bf16_bits_to_f32(got_bits).astype(np.float64)
        want = synth.bf16_bits_to_f32(want_bits).astype(np.float64)
        i = np.argwhere(differ)[0]
        raise AssertionError(f"{differ.sum()} of {differ.size} appended K elements differ; first at {tuple(i)}: "
                             f"{got[tuple(i)]!r} != {want[tuple(i)]!r}")


def check_k_rows_close(got_bits, want_bits):
    """The unfused op sequence (stand-alone norm with a tree sum, rope with sincosf, as the
    reference's own GPU kernels do): every appended K element within one bf16 ulp of the oracle's,
    the ulp taken at max(|want|, 1e-4 * the row's largest magnitude) -- where RoPE's x0*c - x1*s
    cancels, the fp32 rounding of the products is several ulps of the tiny result -- and at most
    0.5 % of the elements different at all."""
    got = synth.bf16_bits_to_f32(got_bits).astype(np.float64)
    want = synth.bf16_bits_to_f32(want_bits).astype(np.float64)
    row_max = np.max(np.abs(want), axis=-1, keepdims=True)
    mag = np.maximum(np.abs(want), 1e-4 * np.maximum(row_max, 1e-30))
    ulp = 2.0 ** (np.floor(np.log2(mag)) - 7)
    excess = np.abs(got - want) / ulp
    assert excess.max() <= 1.0, f"appended K differs by {excess.max():.2f} bf16 ulps"
    assert (got_bits != want_bits).mean() <= 0.005


def fused_once(be, oracle, *, rows, qh, kvh, base, ctx, io, paged, seed, w_q=None, w_k=None, layer=0, layers=1,
               inputs=None, shift=0):
    """Runs one fused step on the device and the oracle's composition on the host.
    Returns (got_out, want_out, got_k_rows, want_k_rows, got_v_rows, want_v_rows).
    shift: the activations (qg, k, v, out) start that many elements into their buffers, so
    that they are not 16-byte aligned."""
    rng = np.random.default_rng(seed)
    if inputs is None:
        qg, k, v = synth.step_inputs(rng, rows, qh, kvh)
        kc = np.zeros((kvh, ctx, 256), np.uint16); vc = np.zeros((kvh, ctx, 256), np.uint16)
        if base:
            kc[:, :base] = synth.cache_bits(rng, kvh, base); vc[:, :base] = synth.cache_bits(rng, kvh, base)
        pos = synth.positions(base, rows)
    else:
        qg, k, v, kc, vc, pos = inputs
    axis, inv = oracle.rope_tables()
    layer_bytes = kvh * ctx * 512
    with Bufs(be) as B:
        el = 2 if io == BF16 else 4
        pad = lambda a: np.concatenate([np.zeros(shift, a.dtype), a.ravel()])
        qgb, _ = B.shared(pad(to_io(qg, io))); kb, _ = B.shared(pad(to_io(k, io))); vb, _ = B.shared(pad(to_io(v, io)))
        ob, ov = B.shared_empty((shift + rows * qh * 256,), io_np(io))
        pb, _ = B.shared(pos); ab, _ = B.shared(axis); fb, _ = B.shared(inv)
        wq = QwRef(B.shared(w_q)[0], 0) if w_q is not None else NULL_REF
        wk = QwRef(B.shared(w_k)[0], 0) if w_k is not None else NULL_REF
        if paged:
            kcb = B.arena(layers, kvh, ctx, seed=seed * 2 + 1); vcb = B.arena(layers, kvh, ctx, seed=seed * 2 + 2)
            if base:
                arena_fill(be, kcb, layer, kc[:, :base], kvh, ctx); arena_fill(be, vcb, layer, vc[:, :base], kvh, ctx)
        else:
            full_k = np.zeros((layers, kvh, ctx, 256), np.uint16); full_v = np.zeros_like(full_k)
            full_k[layer] = kc; full_v[layer] = vc
            kcb = B.device(full_k); vcb = B.device(full_v)
        c = be.cmd_begin()
        ok = be.op_attn_layer_fused(c, QwRef(ob, shift * el), QwRef(qgb, shift * el), QwRef(kb, shift * el), QwRef(vb, shift * el), wq, wk, QwRef(pb, 0),
                                    QwRef(ab, 0), QwRef(fb, 0), QwRef(kcb, layer * layer_bytes),
                                    QwRef(vcb, layer * layer_bytes), rows, qh, kvh, 256, 64, ctx, base, 1e-6, 0.0625, io)
        if not ok:
            err = be.cmd_wait(c, check=False)
            be.cmd_free(c)
            raise AssertionError(f"the fused node declined: {err}")
        be.cmd_wait(c); be.cmd_free(c)
        got = from_io(ov[shift:].reshape(rows, qh, 256), io)
        gk = np.stack([be.kv_read(kcb, layer, h, base, rows, kvh, ctx) for h in range(kvh)])
        gv = np.stack([be.kv_read(vcb, layer, h, base, rows, kvh, ctx) for h in range(kvh)])
        if base:   # history untouched
            assert np.array_equal(be.kv_read(kcb, layer, 0, 0, base, kvh, ctx), kc[0, :base])
    kc2, vc2 = kc.copy(), vc.copy()
    want = oracle.attn_layer(qg, k, v, w_q, w_k, pos, axis, inv, kc2, vc2, rows, qh, kvh, 256, 64, ctx, base, 1e-6,
                             0.0625, ORC_BF16)
    return got, want, gk, kc2[:, base:base + rows], gv, vc2[:, base:base + rows]


@pytest.mark.parametrize("io", [F32, BF16], ids=["f32", "bf16"])
@pytest.mark.parametrize("paged", [False, True], ids=["linear", "arena"])
@pytest.mark.parametrize("rows,qh,kvh,base,ctx", [(1, 16, 4, 0, 128), (1, 16, 4, 333, 512), (1, 24, 4, 2047, 2100),
                                                  (4, 24, 4, 500, 640), (9, 24, 2, 130, 256), (1, 16, 2, 4096, 4200),
                                                  (40, 16, 4, 70, 256), (130, 24, 4, 0, 192)])
def test_fused_matches_oracle(be, oracle, io, paged, rows, qh, kvh, base, ctx):
    w = synth.f32_to_bf16_bits(np.ones(256, np.float32))
    got, want, gk, wk_, gv, wv = fused_once(be, oracle, rows=rows, qh=qh, kvh=kvh, base=base, ctx=ctx, io=io,
                                            paged=paged, seed=rows * 1000 + base, w_q=w, w_k=w)
    assert np.array_equal(gv, wv), "appended V must be bit-exact"
    check_k_rows(gk, wk_)
    assert max_rel_err(got, want) <= 1e-2
    assert rel_l2(got, want) < 6e-3


@pytest.mark.parametrize("fuse_q", [1, 0], ids=["q-in-kernel", "q-in-preop"])
@pytest.mark.parametrize("rows,base", [(300, 0), (200, 77)])
def test_fused_prefill_norm_weights_and_knob(be, oracle, fuse_q, rows, base):
    """Many-row bf16 prefill with non-trivial norm weights, with the query norm + RoPE done by the
    tcgen05 kernel on its own tiles (default) and by the pre-op kernel."""
    rng = np.random.default_rng(11)
    w_q = synth.f32_to_bf16_bits(1.0 + 0.3 * rng.standard_normal(256).astype(np.float32))
    w_k = synth.f32_to_bf16_bits(1.0 + 0.3 * rng.standard_normal(256).astype(np.float32))
    assert be.tune("prefill_fuse_q", fuse_q)
    try:
        got, want, gk, wk_, gv, wv = fused_once(be, oracle, rows=rows, qh=8, kvh=2, base=base, ctx=rows + base + 20,
                                                io=BF16, paged=True, seed=rows + fuse_q, w_q=w_q, w_k=w_k)
    finally:
        be.tune("prefill_fuse_q", 1)
    assert np.array_equal(gv, wv)
    check_k_rows(gk, wk_)
    assert max_rel_err(got, want) <= 1e-2
    assert rel_l2(got, want) < 6e-3


@pytest.mark.parametrize("io", [F32, BF16], ids=["f32", "bf16"])
@pytest.mark.parametrize("rows", [1, 5, 150])
def test_fused_unaligned_activations_are_refused(be, oracle, io, rows):
    """Activations one element into their buffers are not 16-byte aligned: the node declines and
    the command buffer carries an error string -- no launch, no fault, and the backend still works."""
    w = synth.f32_to_bf16_bits(np.ones(256, np.float32))
    with pytest.raises(AssertionError, match="declined.*16-byte aligned"):
        fused_once(be, oracle, rows=rows, qh=8, kvh=2, base=40, ctx=rows + 64, io=io, paged=True, seed=rows + 7,
                   w_q=w, w_k=w, shift=1)
    got, want, *_ = fused_once(be, oracle, rows=rows, qh=8, kvh=2, base=40, ctx=rows + 64, io=io, paged=True,
                               seed=rows + 7, w_q=w, w_k=w, shift=8)
    assert max_rel_err(got, want) <= 1e-2


def test_fused_second_layer_of_arena(be, oracle):
    """Layer addressing by the reference's byte offset into a 3-layer arena."""
    w = synth.f32_to_bf16_bits(1.0 + 0.2 * np.random.default_rng(1).standard_normal(256).astype(np.float32))
    got, want, gk, wk_, gv, wv = fused_once(be, oracle, rows=2, qh=8, kvh=2, base=77, ctx=200, io=F32, paged=True,
                                            seed=5, w_q=w, w_k=None, layer=2, layers=3)
    assert np.array_equal(gv, wv)
    check_k_rows(gk, wk_)
    assert max_rel_err(got, want) <= 1e-2


@pytest.mark.parametrize("case", make_golden.CASES, ids=[c[0] for c in make_golden.CASES])
def test_fused_matches_golden(be, oracle, case):
    """The committed fixtures (outputs of the reference's compiled CPU code) through the fused node."""
    name, rows, qh, kvh, base, ctx, seed, mm = case
    qg, k, v, kc, vc, pos, w = make_golden.case_inputs(rows, qh, kvh, base, ctx, seed, mm, name)
    got, want, gk, _, gv, _ = fused_once(be, oracle, rows=rows, qh=qh, kvh=kvh, base=base, ctx=ctx, io=F32,
                                         paged=False, seed=seed, w_q=w, w_k=w, inputs=(qg, k, v, kc, vc, pos))
    gate = np.ascontiguousarray(qg.reshape(rows, qh, 512)[:, :, 256:])
    want_ref = oracle.mul_sigmoid(GOLDEN[name + "/attn_pre_gate"], gate)
    assert np.array_equal(gv, GOLDEN[name + "/vc_rows"])
    check_k_rows(gk, GOLDEN[name + "/kc_rows"])
    assert max_rel_err(got, want_ref) <= 1e-2
    assert rel_l2(got, want_ref) < 6e-3


def test_fused_equals_unfused_op_sequence(be, oracle):
    """The graph's own sequence of eight ops (qwasar_graph.c:630-659) and the fused node land
    on the same cache rows and, within the bf16-operand tolerance, the same output."""
    rows, qh, kvh, base, ctx = 3, 24, 4, 200, 256
    rng = np.random.default_rng(42)
    qg, k, v = synth.step_inputs(rng, rows, qh, kvh)
    kc = np.zeros((kvh, ctx, 256), np.uint16); vc = np.zeros((kvh, ctx, 256), np.uint16)
    kc[:, :base] = synth.cache_bits(rng, kvh, base); vc[:, :base] = synth.cache_bits(rng, kvh, base)
    pos = synth.positions(base, rows)
    axis, inv = oracle.rope_tables()
    w = synth.f32_to_bf16_bits(np.ones(256, np.float32))
    r = QwRef
    with Bufs(be) as B:
        qgb, _ = B.shared(qg); kb, kv_ = B.shared(k); vb, _ = B.shared(v)
        qb, _ = B.shared_empty((rows, qh, 256), np.float32); gb, _ = B.shared_empty((rows, qh, 256), np.float32)
        ob, ov = B.shared_empty((rows, qh, 256), np.float32)
        pb, _ = B.shared(pos); ab, _ = B.shared(axis); fb, _ = B.shared(inv); wb, _ = B.shared(w)
        kcb, kcv = B.shared(kc); vcb, vcv = B.shared(vc)
        c = be.cmd_begin()
        be.op_split_heads2(c, r(qb, 0), r(gb, 0), r(qgb, 0), rows, qh, 256)
        be.op_rms_norm(c, r(qb, 0), r(qb, 0), r(wb, 0), 256, rows * qh, 1e-6, 1.0)
        be.op_rms_norm(c, r(kb, 0), r(kb, 0), r(wb, 0), 256, rows * kvh, 1e-6, 1.0)
        be.op_rope_partial(c, r(qb, 0), r(pb, 0), r(ab, 0), r(fb, 0), rows, qh, 256, 64)
        be.op_rope_partial(c, r(kb, 0), r(pb, 0), r(ab, 0), r(fb, 0), rows, kvh, 256, 64)
        be.op_kv_write(c, r(kcb, 0), r(vcb, 0), r(kb, 0), r(vb, 0), rows, kvh, 256, ctx, base)
        be.op_attn(c, r(ob, 0), r(qb, 0), r(kcb, 0), r(vcb, 0), rows, qh, kvh, 256, ctx, base, 0.0625)
        be.op_mul_sigmoid(c, r(ob, 0), r(gb, 0), rows * qh * 256)
        be.cmd_wait(c); be.cmd_free(c)
        unfused = np.array(ov); k_unf = np.array(kcv[:, base:base + rows]); v_unf = np.array(vcv[:, base:base + rows])
    got, want, gk, wk_, gv, wv = fused_once(be, oracle, rows=rows, qh=qh, kvh=kvh, base=base, ctx=ctx, io=F32,
                                            paged=True, seed=9, w_q=w, w_k=w, inputs=(qg, k, v, kc, vc, pos))
    assert np.array_equal(v_unf, wv) and np.array_equal(gv, wv)
    check_k_rows_close(k_unf, wk_); check_k_rows(gk, wk_)
    assert max_rel_err(unfused, want) <= 1e-2 and max_rel_err(got, want) <= 1e-2
    assert rel_l2(got, unfused) < 6e-3


@pytest.mark.parametrize("io", [F32, BF16], ids=["f32", "bf16"])
def test_fused_batch_independent_sequences(be, oracle, io):
    """Batched decode: sequences of different depths, each equal to its own single-sequence
    oracle run (the reference has no batch dimension: one session is one sequence)."""
    qh, kvh, ctx, rows = 24, 4, 1536, 1
    depths = [0, 63, 64, 700, 1500, 129, 1024, 31, 5, 999, 1300, 257, 400, 800, 1200, 64, 1, 2, 3]   # 19: two launches
    axis, inv = oracle.rope_tables()
    w = synth.f32_to_bf16_bits(np.ones(256, np.float32))
    rng = np.random.default_rng(123)
    with Bufs(be) as B:
        ab, _ = B.shared(axis); fb, _ = B.shared(inv); wb, _ = B.shared(w)
        outs, qgs, ks, vs, poss, kcs, vcs, host = [], [], [], [], [], [], [], []
        for i, d in enumerate(depths):
            qg, k, v = synth.step_inputs(rng, rows, qh, kvh)
            kc = np.zeros((kvh, ctx, 256), np.uint16); vc = np.zeros((kvh, ctx, 256), np.uint16)
            if d:
                kc[:, :d] = synth.cache_bits(rng, kvh, d); vc[:, :d] = synth.cache_bits(rng, kvh, d)
            ka = B.arena(1, kvh, ctx, seed=i + 1); va = B.arena(1, kvh, ctx, seed=i + 100)
            if d:
                arena_fill(be, ka, 0, kc[:, :d], kvh, ctx); arena_fill(be, va, 0, vc[:, :d], kvh, ctx)
            ob, ov = B.shared_empty((rows, qh, 256), io_np(io))
            outs.append(QwRef(ob, 0)); qgs.append(QwRef(B.shared(to_io(qg, io))[0], 0))
            ks.append(QwRef(B.shared(to_io(k, io))[0], 0)); vs.append(QwRef(B.shared(to_io(v, io))[0], 0))
            poss.append(QwRef(B.shared(synth.positions(d, rows))[0], 0)); kcs.append(QwRef(ka, 0)); vcs.append(QwRef(va, 0))
            host.append((qg, k, v, kc, vc, ov))
        c = be.cmd_begin()
        assert be.op_attn_layer_fused_batch(c, outs, qgs, ks, vs, QwRef(wb, 0), QwRef(wb, 0), poss, QwRef(ab, 0),
                                            QwRef(fb, 0), kcs, vcs, depths, rows, qh, kvh, 256, 64, ctx, 1e-6, 0.0625, io)
        be.cmd_wait(c); be.cmd_free(c)
        for d, (qg, k, v, kc, vc, ov) in zip(depths, host):
            want = oracle.attn_layer(qg, k, v, w, w, synth.positions(d, rows), axis, inv, kc, vc, rows, qh, kvh, 256,
                                     64, ctx, d, 1e-6, 0.0625, ORC_BF16)
            got = from_io(ov, io)
            assert max_rel_err(got, want) <= 1e-2, f"depth {d}"
