"""The five benchmark configurations at their full sizes, against the oracle.

Decode / verify configurations run the whole oracle (seconds on a few cores).  The
4096-row prefill compares a sample of rows (the oracle run as independent single-row
calls, which is the same arithmetic per row: qwasar_cpu.c:364-369) and checks the whole
appended cache."""
import numpy as np
import pytest

from conftest import max_rel_err, rel_l2
from gpu_util import Bufs, QwRef, F32, BF16, to_io, from_io, io_np
from oracle.oracle import BF16 as ORC_BF16
from qwasar_b200 import synth
from test_gpu_fused import check_k_rows

pytestmark = pytest.mark.gpu


def decode_config(be, oracle, name, io, paged):
    cfg = synth.WORKLOADS[name]
    qh, kvh, rows, base = cfg["q_heads"], cfg["kv_heads"], cfg["rows"], cfg["base_pos"]
    ctx = base + rows + 8
    rng = np.random.default_rng(cfg["seed"])
    qg, k, v = synth.step_inputs(rng, rows, qh, kvh)
    kc = np.zeros((kvh, ctx, 256), np.uint16); vc = np.zeros((kvh, ctx, 256), np.uint16)
    kc[:, :base] = synth.cache_bits(rng, kvh, base); vc[:, :base] = synth.cache_bits(rng, kvh, base)
    kc[:, base + rows:] = oracle.to_cache(np.float32([30.0]))[0]     # stale tail, as the reference poisons it
    vc[:, base + rows:] = oracle.to_cache(np.float32([-999.0]))[0]
    pos = synth.positions(base, rows)
    axis, inv = oracle.rope_tables()
    w = synth.f32_to_bf16_bits(np.ones(256, np.float32))
    with Bufs(be) as B:
        qgb, _ = B.shared(to_io(qg, io)); kb, _ = B.shared(to_io(k, io)); vb, _ = B.shared(to_io(v, io))
        ob, ov = B.shared_empty((rows, qh, 256), io_np(io))
        pb, _ = B.shared(pos); ab, _ = B.shared(axis); fb, _ = B.shared(inv); wb, _ = B.shared(w)
        if paged:
            kcb = B.arena(1, kvh, ctx, seed=7); vcb = B.arena(1, kvh, ctx, seed=8)
            for h in range(kvh):
                be.kv_store(kcb, 0, h, 0, kc[h, :base], kvh, ctx); be.kv_store(vcb, 0, h, 0, vc[h, :base], kvh, ctx)
        else:
            kcb = B.device(kc); vcb = B.device(vc)
        c = be.cmd_begin()
        assert be.op_attn_layer_fused(c, QwRef(ob, 0), QwRef(qgb, 0), QwRef(kb, 0), QwRef(vb, 0), QwRef(wb, 0),
                                      QwRef(wb, 0), QwRef(pb, 0), QwRef(ab, 0), QwRef(fb, 0), QwRef(kcb, 0),
                                      QwRef(vcb, 0), rows, qh, kvh, 256, 64, ctx, base, 1e-6, 0.0625, io)
        be.cmd_wait(c); be.cmd_free(c)
        got = from_io(ov, io)
        gk = np.stack([be.kv_read(kcb, 0, h, base, rows, kvh, ctx) for h in range(kvh)])
        gv = np.stack([be.kv_read(vcb, 0, h, base, rows, kvh, ctx) for h in range(kvh)])
    want = oracle.attn_layer(qg, k, v, w, w, pos, axis, inv, kc, vc, rows, qh, kvh, 256, 64, ctx, base, 1e-6, 0.0625,
                             ORC_BF16)
    assert np.array_equal(gv, vc[:, base:base + rows])
    check_k_rows(gk, kc[:, base:base + rows])
    return got, want


@pytest.mark.parametrize("name,io,paged", [("c1_9b_decode_4k", F32, False), ("c1_9b_decode_4k", BF16, True),
                                           ("c3_27b_decode_32k", BF16, True), ("c3_27b_decode_32k", F32, False),
                                           ("c4_27b_verify_32k", BF16, True), ("c4_27b_verify_32k", F32, False),
                                           ("c5_flash_decode_262k", BF16, True)])
def test_decode_configs_full_size(be, oracle, name, io, paged):
    got, want = decode_config(be, oracle, name, io, paged)
    assert max_rel_err(got, want) <= 1e-2, name
    assert rel_l2(got, want) < 6e-3, name


@pytest.mark.parametrize("chunked", [False, True], ids=["one_call", "chunks_of_256"])
def test_prefill_4096_full_size(be, oracle, chunked):
    """Config 2: a 4096-token causal prefill into an empty cache, as one call and as the
    engine's 16 chunks of 256 rows (qwasar_graph.c:1521-1569)."""
    cfg = synth.WORKLOADS["c2_9b_prefill_4k"]
    qh, kvh, rows = cfg["q_heads"], cfg["kv_heads"], cfg["rows"]
    ctx = rows + 8
    rng = np.random.default_rng(cfg["seed"])
    qg, k, v = synth.step_inputs(rng, rows, qh, kvh)
    axis, inv = oracle.rope_tables()
    w = synth.f32_to_bf16_bits(np.ones(256, np.float32))
    io = BF16
    with Bufs(be) as B:
        ab, _ = B.shared(axis); fb, _ = B.shared(inv); wb, _ = B.shared(w)
        qgb = B.device(to_io(qg, io)); kb = B.device(to_io(k, io)); vb = B.device(to_io(v, io))
        pb = B.device(synth.positions(0, rows) if not chunked else
                      np.concatenate([synth.positions(c0, 256).reshape(-1) for c0 in range(0, rows, 256)]))
        ob = B.device(np.zeros((rows, qh, 256), np.uint16))
        kcb = B.arena(1, kvh, ctx, seed=3); vcb = B.arena(1, kvh, ctx, seed=4)
        c = be.cmd_begin()
        step = 256 if chunked else rows
        for c0 in range(0, rows, step):
            assert be.op_attn_layer_fused(
                c, QwRef(ob, c0 * qh * 256 * 2), QwRef(qgb, c0 * qh * 512 * 2), QwRef(kb, c0 * kvh * 256 * 2),
                QwRef(vb, c0 * kvh * 256 * 2), QwRef(wb, 0), QwRef(wb, 0),
                QwRef(pb, (c0 // step) * 3 * step * 4), QwRef(ab, 0), QwRef(fb, 0), QwRef(kcb, 0), QwRef(vcb, 0),
                step, qh, kvh, 256, 64, ctx, c0, 1e-6, 0.0625, io)
        be.cmd_wait(c); be.cmd_free(c)
        got_bits = np.empty((rows, qh, 256), np.uint16); be.buf_download(ob, 0, got_bits)
        got = synth.bf16_bits_to_f32(got_bits)
        gk = np.stack([be.kv_read(kcb, 0, h, 0, rows, kvh, ctx) for h in range(kvh)])
        gv = np.stack([be.kv_read(vcb, 0, h, 0, rows, kvh, ctx) for h in range(kvh)])
    # oracle: pre-ops and append for all rows, attention for a sample of rows
    q_all, gate = oracle.split_heads2(qg, rows, qh, 256)
    q_all = oracle.rms_norm(q_all, w, 256, rows * qh, 1e-6); kk = oracle.rms_norm(k, w, 256, rows * kvh, 1e-6)
    pos = synth.positions(0, rows)
    q_all = oracle.rope_partial(q_all, pos, axis, inv, rows, qh, 256, 64)
    kk = oracle.rope_partial(kk, pos, axis, inv, rows, kvh, 256, 64)
    kc = np.zeros((kvh, ctx, 256), np.uint16); vc = np.zeros((kvh, ctx, 256), np.uint16)
    oracle.kv_write(kc, vc, kk, v, rows, kvh, 256, ctx, 0)
    assert np.array_equal(gv, vc[:, :rows])
    check_k_rows(gk, kc[:, :rows])
    sample = sorted(set([0, 1, 15, 16, 127, 128, 255, 256, 257, 1023, 2048, 4095] +
                        np.random.default_rng(0).integers(0, rows, 20).tolist()))
    for r in sample:
        want = oracle.attn_decode(q_all[r:r + 1], kc, vc, 1, qh, kvh, 256, ctx, r, 0.0625)
        want = oracle.mul_sigmoid(want, gate[r:r + 1])
        assert max_rel_err(got[r:r + 1], want) <= 1e-2, f"row {r}"
        assert rel_l2(got[r:r + 1], want) < 8e-3, f"row {r}"
    assert np.isfinite(got).all()
