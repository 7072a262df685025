"""The KV section of the reference's packed session state over the paged bf16 arena and over a
plain cache buffer: qw_kv_pack / qw_kv_unpack against a numpy restatement of the layout written by
qw_session_pack (qwasar_graph.c:296-303, 332-339: layer by layer, head by head, the K rows of the
used positions, then the V rows) and read back by qw_session_unpack (:352-373).  Integer work:
every comparison is bit-exact."""
import numpy as np
import pytest

from gpu_util import Bufs, QwRef, BF16, arena_fill
from qwasar_b200 import synth

pytestmark = pytest.mark.gpu


def packed_reference(kc, vc, n):
    """kc, vc: uint16 [layers, kv_heads, ctx, 256] -> [layers, kv_heads, 2, n, 256]."""
    return np.stack([kc[:, :, :n], vc[:, :, :n]], axis=2)


def make_caches(B, be, layers, kvh, ctx, n, paged, seed):
    rng = np.random.default_rng(seed)
    kc = np.zeros((layers, kvh, ctx, 256), np.uint16); vc = np.zeros_like(kc)
    kc[:, :, :n] = rng.integers(0, 0x7F80, (layers, kvh, n, 256), dtype=np.uint16)
    vc[:, :, :n] = rng.integers(0, 0x7F80, (layers, kvh, n, 256), dtype=np.uint16)
    if paged:
        kb = B.arena(layers, kvh, ctx, seed=seed + 1); vb = B.arena(layers, kvh, ctx, seed=seed + 2)
        for l in range(layers):
            if n:
                arena_fill(be, kb, l, kc[l, :, :n], kvh, ctx); arena_fill(be, vb, l, vc[l, :, :n], kvh, ctx)
    else:
        kb = B.device(kc); vb = B.device(vc)
    return kc, vc, kb, vb


@pytest.mark.parametrize("paged", [True, False], ids=["arena", "linear"])
@pytest.mark.parametrize("layers,kvh,ctx,n", [(1, 1, 64, 1), (2, 4, 300, 130), (3, 2, 257, 257), (2, 2, 128, 64)])
def test_pack_matches_reference_layout(be, paged, layers, kvh, ctx, n):
    with Bufs(be) as B:
        kc, vc, kb, vb = make_caches(B, be, layers, kvh, ctx, n, paged, seed=layers * 100 + n)
        got = be.kv_pack(kb, vb, layers, kvh, ctx, n)
        assert np.array_equal(got, packed_reference(kc, vc, n))
        # a shorter prefix of the same caches is the same bytes, compacted
        if n > 1:
            m = n // 2
            assert np.array_equal(be.kv_pack(kb, vb, layers, kvh, ctx, m), packed_reference(kc, vc, m))


@pytest.mark.parametrize("paged_src,paged_dst", [(True, True), (True, False), (False, True)],
                         ids=["arena-arena", "arena-linear", "linear-arena"])
def test_unpack_restores_bit_identically(be, paged_src, paged_dst):
    layers, kvh, ctx, n = 2, 4, 400, 333
    with Bufs(be) as B:
        kc, vc, kb, vb = make_caches(B, be, layers, kvh, ctx, n, paged_src, seed=7)
        state = be.kv_pack(kb, vb, layers, kvh, ctx, n)
        ctx2 = 512                                             # a checkpoint is portable across context sizes
        if paged_dst:
            k2 = B.arena(layers, kvh, ctx2, seed=91); v2 = B.arena(layers, kvh, ctx2, seed=92)
        else:
            k2 = B.device(np.zeros((layers, kvh, ctx2, 256), np.uint16)); v2 = B.device(np.zeros((layers, kvh, ctx2, 256), np.uint16))
        be.kv_unpack(k2, v2, state, ctx2)
        for l in range(layers):
            for h in range(kvh):
                assert np.array_equal(be.kv_read(k2, l, h, 0, n, kvh, ctx2), kc[l, h, :n])
                assert np.array_equal(be.kv_read(v2, l, h, 0, n, kvh, ctx2), vc[l, h, :n])
        assert np.array_equal(be.kv_pack(k2, v2, layers, kvh, ctx2, n), state)


def test_decode_continues_from_a_restored_arena(be, oracle):
    """Prefill 40 tokens, checkpoint, restore into fresh arenas, decode one token there: the same
    output as decoding on the original arenas, bit for bit."""
    rows, qh, kvh, ctx = 40, 8, 2, 128
    rng = np.random.default_rng(3)
    qg, k, v = synth.step_inputs(rng, rows, qh, kvh)
    qg1, k1, v1 = synth.step_inputs(rng, 1, qh, kvh)
    axis, inv = oracle.rope_tables()
    w = synth.f32_to_bf16_bits(np.ones(256, np.float32))

    def step(B, kb, vb, qg_, k_, v_, n_rows, base):
        bufs = [B.shared(synth.f32_to_bf16_bits(a))[0] for a in (qg_, k_, v_)]
        ob, ov = B.shared_empty((n_rows, qh, 256), np.uint16)
        pb, _ = B.shared(synth.positions(base, n_rows)); ab, _ = B.shared(axis); fb, _ = B.shared(inv); wb, _ = B.shared(w)
        c = be.cmd_begin()
        assert be.op_attn_layer_fused(c, QwRef(ob, 0), QwRef(bufs[0], 0), QwRef(bufs[1], 0), QwRef(bufs[2], 0), QwRef(wb, 0),
                                      QwRef(wb, 0), QwRef(pb, 0), QwRef(ab, 0), QwRef(fb, 0), QwRef(kb, 0), QwRef(vb, 0),
                                      n_rows, qh, kvh, 256, 64, ctx, base, 1e-6, 0.0625, BF16)
        be.cmd_wait(c); be.cmd_free(c)
        return np.array(ov)

    with Bufs(be) as B:
        ka = B.arena(1, kvh, ctx, seed=5); va = B.arena(1, kvh, ctx, seed=6)
        step(B, ka, va, qg, k, v, rows, 0)
        state = be.kv_pack(ka, va, 1, kvh, ctx, rows)
        kb = B.arena(1, kvh, ctx, seed=15); vb = B.arena(1, kvh, ctx, seed=16)
        be.kv_unpack(kb, vb, state, ctx)
        out_a = step(B, ka, va, qg1, k1, v1, 1, rows)
        out_b = step(B, kb, vb, qg1, k1, v1, 1, rows)
        assert np.array_equal(out_a, out_b)


def test_wrong_length_is_refused(be):
    with Bufs(be) as B:
        kb = B.arena(1, 2, 64, seed=1); vb = B.arena(1, 2, 64, seed=2)
        buf = np.zeros(10, np.uint16)
        assert not be.lib.qw_kv_unpack(kb, vb, 1, 2, 64, 256, 8, buf.ctypes.data, buf.nbytes)
        assert "bytes given" in be.last_error()
        assert not be.lib.qw_kv_pack(kb, vb, 1, 2, 64, 256, 8, buf.ctypes.data, buf.nbytes)
