"""Sequence split: per-range partials (qw_op_attn_partial) merged by qw_op_attn_merge equal
the unsplit attention -- the single-GPU statement of the multi-GPU path (each rank computes
one range, the partials are all-gathered, every rank merges)."""
import numpy as np
import pytest

from conftest import max_rel_err, rel_l2
from gpu_util import Bufs, QwRef, F32, BF16
from qwasar_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,qh,kvh,base,cuts", [
    (1, 16, 2, 5000, [0, 1280, 2560, 3840, 5001]),
    (1, 24, 4, 777, [0, 64, 128, 778]),
    (4, 24, 4, 1000, [0, 512, 1004]),
    (1, 16, 2, 300, [0, 320, 640, 960]),          # ranges past the end: empty partials drop out
])
def test_partials_merge_to_whole(be, oracle, rows, qh, kvh, base, cuts):
    ctx = base + rows + 3
    rng = np.random.default_rng(base)
    q = synth.normal_bf16(rng, (rows, qh, 256))
    gate = synth.normal_bf16(rng, (rows, qh, 256))
    kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
    parts = len(cuts) - 1
    n_rh = rows * qh
    with Bufs(be) as B:
        qb, _ = B.shared(q); gb, _ = B.shared(gate)
        kcb = B.device(kc); vcb = B.device(vc)
        pa, pav = B.shared_empty((parts, n_rh, 256), np.float32); ps, psv = B.shared_empty((parts, n_rh, 2), np.float32)
        ob, ov = B.shared_empty((rows, qh, 256), np.float32)
        c = be.cmd_begin()
        for i in range(parts):
            assert be.op_attn_partial(c, QwRef(pa, i * n_rh * 256 * 4), QwRef(ps, i * n_rh * 2 * 4), QwRef(qb, 0),
                                      QwRef(kcb, 0), QwRef(vcb, 0), rows, qh, kvh, 256, ctx, base, cuts[i],
                                      cuts[i + 1], 0.0625, F32)
        be.op_attn_merge(c, QwRef(ob, 0), QwRef(pa, 0), QwRef(ps, 0), QwRef(gb, 0), rows, qh, 256, parts, 256, F32, F32, 0)
        be.cmd_wait(c); be.cmd_free(c)
        got = np.array(ov); stats = np.array(psv)
    want = oracle.mul_sigmoid(oracle.attn_decode(q, kc, vc, rows, qh, kvh, 256, ctx, base, 0.0625), gate)
    assert max_rel_err(got, want) <= 1e-2 and rel_l2(got, want) < 6e-3
    # a range wholly past the visible keys contributes sum 0
    for i in range(parts):
        if cuts[i] >= base + rows:
            assert np.all(stats[i, :, 1] == 0.0)
    # each partial is the oracle's partial of that range (row 0, head 0)
    for i in range(parts):
        hi = min(cuts[i + 1], base + 1)
        acc, st = oracle.attn_partial(q[0, 0], kc[0], vc[0], cuts[i], hi, 256, 0.0625)
        if st[1] > 0:
            # compare the normalised partial (the max each side subtracts may differ)
            assert rel_l2(np.array(pav[i, 0]) / stats[i, 0, 1], acc / st[1]) < 6e-3


def test_cuts_from_seq_range_at_an_unaligned_length(be, oracle):
    """Trailing shards of a short sequence are empty and start where the keys end, which need not be
    a multiple of 64 (sharding.seq_range): the op takes them and leaves an empty partial."""
    from qwasar_b200 import sharding
    rows, qh, kvh, base, shards = 1, 16, 2, 99, 4          # 100 keys
    ctx = base + rows + 3
    rng = np.random.default_rng(4)
    q = synth.normal_bf16(rng, (rows, qh, 256)); gate = synth.normal_bf16(rng, (rows, qh, 256))
    kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
    n_rh = rows * qh
    with Bufs(be) as B:
        qb, _ = B.shared(q); gb, _ = B.shared(gate)
        kcb = B.device(kc); vcb = B.device(vc)
        pa, _ = B.shared_empty((shards, n_rh, 256), np.float32); ps, psv = B.shared_empty((shards, n_rh, 2), np.float32)
        ob, ov = B.shared_empty((rows, qh, 256), np.float32)
        c = be.cmd_begin()
        for i in range(shards):
            lo, hi = sharding.seq_range(i, shards, base + rows)
            assert be.op_attn_partial(c, QwRef(pa, i * n_rh * 256 * 4), QwRef(ps, i * n_rh * 2 * 4), QwRef(qb, 0), QwRef(kcb, 0),
                                      QwRef(vcb, 0), rows, qh, kvh, 256, ctx, base, lo, hi, 0.0625, F32), (i, lo, hi)
        be.op_attn_merge(c, QwRef(ob, 0), QwRef(pa, 0), QwRef(ps, 0), QwRef(gb, 0), rows, qh, 256, shards, 256, F32, F32, 0)
        be.cmd_wait(c); be.cmd_free(c)
        assert np.all(np.array(psv)[2:, :, 1] == 0.0)
        got = np.array(ov)
    want = oracle.mul_sigmoid(oracle.attn_decode(q, kc, vc, rows, qh, kvh, 256, ctx, base, 0.0625), gate)
    assert max_rel_err(got, want) <= 1e-2
