"""The 4-bit affine product (qwasar_gpu.h:84-118) against the oracle, with the reference's own
error measure and bound for its fp32 kernel (tests/test_qmv.c:31-50, 129): per output,
|double-precision dot over the dequantised row - got| / sum of the absolute terms < 2e-6."""
import ctypes as C

import numpy as np
import pytest

from gpu_util import Bufs, QwRef
from qwasar_b200 import synth

pytestmark = pytest.mark.gpu


def q4_weights(rng, n, k, group):
    w = rng.integers(0, 2 ** 32, (n, k // 8), dtype=np.uint64).astype(np.uint32)
    sc = synth.f32_to_bf16_bits((0.02 * rng.standard_normal((n, k // group))).astype(np.float32))
    bi = synth.f32_to_bf16_bits((0.1 * rng.standard_normal((n, k // group))).astype(np.float32))
    return w, sc, bi


def dequant(w, sc, bi, k, group):
    nib = ((w[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).reshape(w.shape[0], k).astype(np.float32)
    s = np.repeat(synth.bf16_bits_to_f32(sc), group, axis=1); b = np.repeat(synth.bf16_bits_to_f32(bi), group, axis=1)
    return s * nib + b


def worst_rel_err(got, x, deq):
    terms = deq[None, :, :].astype(np.float64) * x[:, None, :].astype(np.float64)      # [rows, n, k]
    return float(np.max(np.abs(terms.sum(-1) - got) / np.maximum(np.abs(terms).sum(-1), 1e-300)))


@pytest.mark.parametrize("op", ["op_qmat_q4", "op_qmv_q4", "op_qmm_q4"])
@pytest.mark.parametrize("k,n,rows,group", [(64, 3, 1, 64), (4096, 48, 1, 64), (8192, 70, 2, 64), (5120, 33, 1, 32), (2048, 1000, 5, 64), (1024, 100, 17, 32), (256, 9, 8, 32),
                                              (5120, 12288, 1, 64), (5120, 1000, 2, 64), (12288, 500, 1, 64), (4096, 257, 2, 64), (128, 16, 1, 64),
                                              (640, 1, 1, 64), (16384, 40, 2, 64),
                                              (2048, 256, 16, 64), (1024, 520, 200, 64), (5120, 768, 300, 64), (2048, 1000, 129, 64), (2560, 8, 16, 64), (6144, 264, 64, 64), (2048, 100, 15, 64), (1024, 72, 7, 64),
                                              (5120, 1000, 3, 64), (5120, 2000, 4, 64), (6144, 264, 4, 64), (512, 50, 3, 64), (7168, 40, 4, 64), (8192, 70, 4, 64),
                                              (3072, 17, 4, 64), (5120, 300, 11, 64),
                                              (4608, 40, 1, 64), (3584, 24, 2, 64), (1536, 33, 1, 64), (5632, 50, 3, 64), (5632, 48, 1, 64)])
def test_q4_product(be, oracle, op, k, n, rows, group):
    rng = np.random.default_rng(k + n + rows)
    w, sc, bi = q4_weights(rng, n, k, group)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    with Bufs(be) as B:
        xb, _ = B.shared(x); wb, _ = B.shared(w); sb, _ = B.shared(sc); bb, _ = B.shared(bi)
        yb, yv = B.shared_empty((rows, n), np.float32, fill=np.float32(np.nan))
        c = be.cmd_begin()
        getattr(be, op)(c, QwRef(yb, 0), QwRef(xb, 0), QwRef(wb, 0), QwRef(sb, 0), QwRef(bb, 0), k, n, rows, group)
        be.cmd_wait(c); be.cmd_free(c)
        got = np.array(yv)
    assert np.all(np.isfinite(got))
    # 16 rows and more of a 64-group product with k a multiple of 512 from 2048 up (the model's shapes, where the
    # reference's bound for its tensor form holds, tests/test_qmv.c:117-131; the error falls with the square root of k)
    # run on the tensor cores with fp16 operands; everything else is fp32 or exact integers
    tensor_form = rows >= 16 and group == 64 and k % 512 == 0 and k >= 2048 and n % 8 == 0
    assert worst_rel_err(got, x, dequant(w, sc, bi, k, group)) < (5e-5 if tensor_form else 2e-6)
    if k * n * rows <= 2_000_000:                                # and the oracle itself, to the same measure
        want = oracle.qmv_q4(x, w, sc, bi, k, n, rows, group)
        assert worst_rel_err(want, x, dequant(w, sc, bi, k, group)) < 2e-5
        assert np.allclose(got, want, rtol=0, atol=(1e-3 if tensor_form else 2e-5) * np.abs(want).max() + 1e-6)


@pytest.mark.parametrize("rows", [2, 4, 3])
@pytest.mark.parametrize("kind", ["positive", "outlier", "tiny", "huge", "zero", "nan"])
def test_q4_product_input_ranges(be, kind, rows):
    """The product of up to four tokens turns x into scaled integers, each token by its own scale:
    inputs that stress the scale -- one-signed (nothing cancels in the sums), a 1e4 outlier over unit
    noise, magnitudes near the ends of the fp32 range, all zeros -- stay inside the reference's
    bound; a NaN in one token poisons that token's outputs and leaves the other tokens' alone."""
    k, n, group = 5120, 300, 64
    rng = np.random.default_rng(len(kind))
    w, sc, bi = q4_weights(rng, n, k, group)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    if kind == "positive":
        x = np.abs(x) + 1.0
    elif kind == "outlier":
        x[0, 77] = 1.0e4; x[1, 4000] = -3.0e4; x[rows - 1, 5119] = 2.0e4
    elif kind == "tiny":
        x *= np.float32(1e-30)
    elif kind == "huge":
        x *= np.float32(1e30)
    elif kind == "zero":
        x[0] = 0.0
    elif kind == "nan":
        x[1, 123] = np.nan
    with Bufs(be) as B:
        xb, _ = B.shared(x); wb, _ = B.shared(w); sb, _ = B.shared(sc); bb, _ = B.shared(bi)
        yb, yv = B.shared_empty((rows, n), np.float32, fill=np.float32(7.0))
        c = be.cmd_begin()
        be.op_qmat_q4(c, QwRef(yb, 0), QwRef(xb, 0), QwRef(wb, 0), QwRef(sb, 0), QwRef(bb, 0), k, n, rows, group)
        be.cmd_wait(c); be.cmd_free(c)
        got = np.array(yv)
    deq = dequant(w, sc, bi, k, group)
    if kind == "nan":
        keep = [r for r in range(rows) if r != 1]
        assert np.all(np.isnan(got[1])) and np.all(np.isfinite(got[keep]))
        assert worst_rel_err(got[keep], x[keep], deq) < 2e-6
        return
    assert np.all(np.isfinite(got))
    if kind == "zero":
        assert np.all(got[0] == 0.0)
        assert worst_rel_err(got[1:], x[1:], deq) < 2e-6
        return
    with np.errstate(over="ignore"):
        assert worst_rel_err(got, x, deq) < 2e-6


def test_q4_many_tokens_forms_agree(be):
    """The tensor-core form against the fp32 kernel on the same operands (`qmm_tc` 1 | 0), ragged edges in rows and n."""
    k, n, rows, group = 2560, 776, 333, 64
    rng = np.random.default_rng(99)
    w, sc, bi = q4_weights(rng, n, k, group)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    outs = []
    try:
        for knob in (1, 0):
            assert be.tune("qmm_tc", knob)
            with Bufs(be) as B:
                xb, _ = B.shared(x); wb, _ = B.shared(w); sb, _ = B.shared(sc); bb, _ = B.shared(bi)
                yb, yv = B.shared_empty((rows, n), np.float32, fill=np.float32(np.nan))
                c = be.cmd_begin()
                be.op_qmm_q4(c, QwRef(yb, 0), QwRef(xb, 0), QwRef(wb, 0), QwRef(sb, 0), QwRef(bb, 0), k, n, rows, group)
                be.cmd_wait(c); be.cmd_free(c)
                outs.append(np.array(yv))
    finally:
        be.tune("qmm_tc", 1)
    deq = dequant(w, sc, bi, k, group)
    assert worst_rel_err(outs[0], x, deq) < 5e-5 and worst_rel_err(outs[1], x, deq) < 2e-6
    assert np.max(np.abs(outs[0] - outs[1])) < 5e-5 * np.max(np.abs(deq).astype(np.float64) @ np.abs(x).astype(np.float64).T)


def test_q4_multi(be, oracle):
    """Up to four one-token products sharing x (qwasar_gpu.h:105-109); k < 2048 is declined."""
    from qwasar_b200.backend import QwRef as Ref

    class Part(C.Structure):
        _fields_ = [("y", Ref), ("w", Ref), ("scales", Ref), ("biases", Ref), ("n", C.c_int32)]
    rng = np.random.default_rng(4)
    k, group, ns = 2048, 64, [48, 7, 130]
    x = rng.standard_normal((1, k)).astype(np.float32)
    with Bufs(be) as B:
        xb, _ = B.shared(x)
        parts, outs, wts = (Part * len(ns))(), [], []
        for i, n in enumerate(ns):
            w, sc, bi = q4_weights(rng, n, k, group)
            wb, _ = B.shared(w); sb, _ = B.shared(sc); bb, _ = B.shared(bi)
            yb, yv = B.shared_empty((1, n), np.float32, fill=np.float32(np.nan))
            parts[i] = Part(Ref(yb, 0), Ref(wb, 0), Ref(sb, 0), Ref(bb, 0), n)
            outs.append(yv); wts.append((w, sc, bi))
        c = be.cmd_begin()
        n0 = be.launch_count()
        assert be.lib.qw_op_qmv_q4_multi(c, Ref(xb, 0), k, group, len(ns), C.addressof(parts))
        assert be.launch_count() - n0 == 1, "the parts share one dispatch (qwasar_gpu.h:105-109)"
        assert not be.lib.qw_op_qmv_q4_multi(c, Ref(xb, 0), 1024, group, len(ns), C.addressof(parts))
        be.cmd_wait(c); be.cmd_free(c)
        for yv, (w, sc, bi) in zip(outs, wts):
            assert worst_rel_err(np.array(yv), x, dequant(w, sc, bi, k, group)) < 2e-6
