"""Arenas that share one page pool (the layout for serving many sequences on one GPU): logical
contents stay those of the head-major array, one attention launch carries every sequence of the
pool, pages return to the pool when an arena is freed."""
import numpy as np
import pytest

from conftest import max_rel_err
from gpu_util import Bufs, QwRef, BF16, F32, to_io, from_io, io_np, arena_fill, arena_read
from oracle.oracle import BF16 as ORC_BF16
from qwasar_b200 import synth

pytestmark = pytest.mark.gpu


def test_forty_sequences_of_one_pool_take_one_launch_of_each_kernel(be, oracle):
    """40 independent one-token decode steps whose K and V arenas all live in one pool: the pre-op,
    the split-KV kernel and the merge each launch once, every sequence equals its own oracle run
    and the appended rows are bit-exact."""
    qh, kvh, ctx, rows, io = 8, 2, 1300, 1, BF16
    n_seq = 40
    rng = np.random.default_rng(77)
    depths = [int(d) for d in rng.integers(0, 1200, n_seq)]
    depths[0], depths[1] = 0, 1199
    axis, inv = oracle.rope_tables()
    w = synth.f32_to_bf16_bits(np.ones(256, np.float32))
    pool = be.kv_pool_alloc(2 * n_seq * kvh * ((ctx + 63) // 64) * 32768, shuffle_seed=9)
    with Bufs(be) as B:
        ab, _ = B.shared(axis); fb, _ = B.shared(inv); wb, _ = B.shared(w)
        outs, qgs, ks, vs, poss, kcs, vcs, host = [], [], [], [], [], [], [], []
        for d in depths:
            qg, k, v = synth.step_inputs(rng, rows, qh, kvh)
            kc = np.zeros((kvh, ctx, 256), np.uint16); vc = np.zeros((kvh, ctx, 256), np.uint16)
            ka = be.kv_arena_alloc_in(pool, 1, kvh, ctx); va = be.kv_arena_alloc_in(pool, 1, kvh, ctx)
            B.all += [ka, va]
            if d:
                kc[:, :d] = synth.cache_bits(rng, kvh, d); vc[:, :d] = synth.cache_bits(rng, kvh, d)
                arena_fill(be, ka, 0, kc[:, :d], kvh, ctx); arena_fill(be, va, 0, vc[:, :d], kvh, ctx)
            ob, ov = B.shared_empty((rows, qh, 256), io_np(io))
            outs.append(QwRef(ob, 0)); qgs.append(QwRef(B.shared(to_io(qg, io))[0], 0))
            ks.append(QwRef(B.shared(to_io(k, io))[0], 0)); vs.append(QwRef(B.shared(to_io(v, io))[0], 0))
            poss.append(QwRef(B.shared(synth.positions(d, rows))[0], 0)); kcs.append(QwRef(ka, 0)); vcs.append(QwRef(va, 0))
            host.append((qg, k, v, kc, vc, ov, ka, va))
        n0 = be.launch_count()
        c = be.cmd_begin()
        assert be.op_attn_layer_fused_batch(c, outs, qgs, ks, vs, QwRef(wb, 0), QwRef(wb, 0), poss, QwRef(ab, 0),
                                            QwRef(fb, 0), kcs, vcs, depths, rows, qh, kvh, 256, 64, ctx, 1e-6, 0.0625, io)
        be.cmd_wait(c); be.cmd_free(c)
        assert be.launch_count() - n0 == 3, "one pre-op, one split-KV, one merge launch for the whole batch"
        for d, (qg, k, v, kc, vc, ov, ka, va) in zip(depths, host):
            want = oracle.attn_layer(qg, k, v, w, w, synth.positions(d, rows), axis, inv, kc, vc, rows, qh, kvh, 256,
                                     64, ctx, d, 1e-6, 0.0625, ORC_BF16)
            assert max_rel_err(from_io(ov, io), want) <= 1e-2, f"depth {d}"
            assert np.array_equal(arena_read(be, ka, 0, d + 1, kvh, ctx), kc[:, :d + 1]), "K rows, appended one included"
            assert np.array_equal(arena_read(be, va, 0, d + 1, kvh, ctx), vc[:, :d + 1])
        assert be.kv_pool_bytes_committed(pool) > 0
    be.buf_free(pool)


def test_pages_return_to_the_pool(be):
    kvh, ctx = 2, 640
    pool = be.kv_pool_alloc(64 << 20)
    rows = synth.cache_bits(np.random.default_rng(1), kvh, 640)
    a = be.kv_arena_alloc_in(pool, 1, kvh, ctx)
    arena_fill(be, a, 0, rows, kvh, ctx)
    assert be.kv_arena_pages_in_use(a) == kvh * 10
    committed = be.kv_pool_bytes_committed(pool)
    be.buf_free(a)
    b = be.kv_arena_alloc_in(pool, 1, kvh, ctx)
    arena_fill(be, b, 0, rows[:, :100], kvh, ctx)
    assert be.kv_pool_bytes_committed(pool) == committed, "the second arena reuses the first one's pages"
    assert np.array_equal(arena_read(be, b, 0, 100, kvh, ctx), rows[:, :100])
    be.buf_free(pool)          # the handle may go first: the memory stays until the last arena is freed
    assert np.array_equal(arena_read(be, b, 0, 100, kvh, ctx), rows[:, :100])
    be.buf_free(b)


def test_twelve_plain_caches_in_one_call(be, oracle):
    """Plain cache buffers have a tensor map each and a launch holds eight: a batch over twelve
    buffers is split into launches without the caller noticing."""
    qh, kvh, ctx, rows, base = 8, 2, 200, 1, 150
    rng = np.random.default_rng(5)
    with Bufs(be) as B:
        outs, qs, kcs, vcs, host = [], [], [], [], []
        for i in range(12):
            q = synth.normal_bf16(rng, (rows, qh, 256))
            kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
            ob, ov = B.shared_empty((rows, qh, 256), np.float32)
            outs.append(QwRef(ob, 0)); qs.append(QwRef(B.shared(q)[0], 0))
            kcs.append(QwRef(B.device(kc), 0)); vcs.append(QwRef(B.device(vc), 0))
            host.append((q, kc, vc, ov))
        c = be.cmd_begin()
        assert be.op_attn_batch(c, outs, qs, kcs, vcs, [base] * 12, rows, qh, kvh, 256, ctx, 0.0625, F32)
        be.cmd_wait(c); be.cmd_free(c)
        for q, kc, vc, ov in host:
            want = oracle.attn_decode(q, kc, vc, rows, qh, kvh, 256, ctx, base, 0.0625)
            assert max_rel_err(np.array(ov), want) <= 1e-2
