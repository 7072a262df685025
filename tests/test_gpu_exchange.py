"""The exchange of softmax partials between the GPUs of a split sequence (qw_op_attn_exchange),
on ONE device: each "rank" owns an exchange object and a range of positions; all ranks publish
(phase 1), then all collect (phase 2), in one stream, so no kernel ever waits for one launched
after it.  The arithmetic, the addressing of the gather buffers and flags, the empty range and the
bounded wait are what a multi-GPU run uses; there the two phases run as one call per rank."""
import numpy as np
import pytest

from conftest import max_rel_err, rel_l2
from gpu_util import Bufs, QwRef, F32, BF16, NULL_REF
from qwasar_b200 import sharding, synth

pytestmark = pytest.mark.gpu


def make_ranks(be, n, max_rh):
    xs = [be.xchg_create(n, r, max_rh) for r in range(n)]
    for a in range(n):
        for b in range(n):
            if a != b:
                assert be.xchg_attach_local(xs[a], b, xs[b])
    return xs


@pytest.mark.parametrize("rows,qh,kvh,base,n_ranks", [(1, 16, 2, 5000, 4), (1, 16, 2, 700, 8), (4, 24, 4, 1000, 2),
                                                      (1, 16, 2, 100, 4)])     # 100 keys over 4 ranks: two ranks are empty
def test_every_rank_ends_with_the_whole_result(be, oracle, rows, qh, kvh, base, n_ranks):
    ctx = base + rows + 3
    rng = np.random.default_rng(base + n_ranks)
    q = synth.normal_bf16(rng, (rows, qh, 256)); gate = synth.normal_bf16(rng, (rows, qh, 256))
    kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
    want = oracle.mul_sigmoid(oracle.attn_decode(q, kc, vc, rows, qh, kvh, 256, ctx, base, 0.0625), gate)
    xs = make_ranks(be, n_ranks, rows * qh)
    with Bufs(be) as B:
        qb, _ = B.shared(q); gb, _ = B.shared(gate)
        kcb = B.device(kc); vcb = B.device(vc)
        outs = [B.shared_empty((rows, qh, 256), np.float32, fill=-5.0) for _ in range(n_ranks)]
        for epoch in range(3):                       # the slots alternate between two parities: go round more than once
            c = be.cmd_begin()
            for phase in (1, 2):
                for r in range(n_ranks):
                    lo, hi = sharding.seq_range(r, n_ranks, base + rows)
                    assert be.op_attn_exchange(c, xs[r], phase, QwRef(outs[r][0], 0), QwRef(gb, 0), QwRef(qb, 0), QwRef(kcb, 0),
                                               QwRef(vcb, 0), rows, qh, kvh, 256, ctx, base, lo, hi, 0.0625, F32, F32, F32, 256), \
                        be.cmd_error(c)
            be.cmd_wait(c); be.cmd_free(c)
            for r in range(n_ranks):
                got = np.array(outs[r][1])
                assert max_rel_err(got, want) <= 1e-2 and rel_l2(got, want) < 6e-3, f"rank {r}, epoch {epoch}"
                outs[r][1][...] = -5.0
    for x in xs:
        be.xchg_free(x)


def test_batch_of_sequences_of_different_lengths(be, oracle):
    """Three sequences in one round: for the shortest some ranks hold no key at all, so one call
    mixes ranks that stream keys with ranks that only publish an empty record."""
    rows, qh, kvh, n_ranks = 1, 16, 2, 4
    bases = [900, 70, 2000]
    ctx = 2100
    rng = np.random.default_rng(12)
    host = []
    for b in bases:
        q = synth.normal_bf16(rng, (rows, qh, 256)); gate = synth.normal_bf16(rng, (rows, qh, 256))
        kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
        host.append((q, gate, kc, vc, oracle.mul_sigmoid(oracle.attn_decode(q, kc, vc, rows, qh, kvh, 256, ctx, b, 0.0625), gate)))
    xs = make_ranks(be, n_ranks, len(bases) * rows * qh)
    with Bufs(be) as B:
        qs = [QwRef(B.shared(h[0])[0], 0) for h in host]; gs = [QwRef(B.shared(h[1])[0], 0) for h in host]
        kcs = [QwRef(B.device(h[2]), 0) for h in host]; vcs = [QwRef(B.device(h[3]), 0) for h in host]
        outs = [[B.shared_empty((rows, qh, 256), np.float32, fill=-5.0) for _ in bases] for _ in range(n_ranks)]
        # every rank owns the same absolute positions of every sequence: a quarter of the longest
        span = 512
        c = be.cmd_begin()
        for phase in (1, 2):
            for r in range(n_ranks):
                lo = [min(b + rows, r * span) for b in bases]
                hi = [min(b + rows, (r + 1) * span) if r < n_ranks - 1 else b + rows for b in bases]
                lo = [l if l < h else h for l, h in zip(lo, hi)]
                assert be.op_attn_exchange_batch(c, xs[r], phase, [QwRef(o[0], 0) for o in outs[r]], gs, qs, kcs, vcs, bases, lo, hi,
                                                 rows, qh, kvh, 256, ctx, 0.0625, F32, F32, F32, 256), be.cmd_error(c)
        be.cmd_wait(c); be.cmd_free(c)
        for r in range(n_ranks):
            for i, h in enumerate(host):
                assert max_rel_err(np.array(outs[r][i][1]), h[4]) <= 1e-2, f"rank {r}, sequence {i}"
    for x in xs:
        be.xchg_free(x)


def test_a_rank_whose_peer_never_publishes_gives_up_with_an_error(be):
    """The wait for the other ranks' records is bounded: with a 50 ms limit and a peer that never
    runs, the command buffer reports the timeout, writes nothing, and the backend stays usable."""
    rows, qh, kvh, base = 1, 16, 2, 300
    ctx = base + 8
    rng = np.random.default_rng(3)
    q = synth.normal_bf16(rng, (rows, qh, 256))
    kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
    xs = make_ranks(be, 2, rows * qh)
    be.xchg_set_timeout_ms(xs[0], 50)
    with Bufs(be) as B:
        qb, _ = B.shared(q)
        kcb = B.device(kc); vcb = B.device(vc)
        ob, ov = B.shared_empty((rows, qh, 256), np.float32, fill=-5.0)
        c = be.cmd_begin()
        assert be.op_attn_exchange(c, xs[0], 0, QwRef(ob, 0), NULL_REF, QwRef(qb, 0), QwRef(kcb, 0), QwRef(vcb, 0), rows, qh, kvh,
                                   256, ctx, base, 0, 192, 0.0625, F32, F32, F32, 256)
        err = be.cmd_wait(c, check=False)
        be.cmd_free(c)
        assert err and "did not arrive" in err
        assert np.all(np.array(ov) == -5.0)
        # the next command buffer is clean, and ordinary work runs
        c = be.cmd_begin()
        assert be.op_attn_decode_tensor(c, QwRef(ob, 0), QwRef(qb, 0), QwRef(kcb, 0), QwRef(vcb, 0), rows, qh, kvh, 256, ctx, base, 0.0625)
        assert be.cmd_wait(c, check=False) is None
        be.cmd_free(c)
    for x in xs:
        be.xchg_free(x)
