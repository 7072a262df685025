"""QSA's indexer ops (qwasar_gpu.h:620-641) against the oracle, in the shape of the reference's own
test (tests/test_sparse.c:348-470): block scores within 1e-4 of the CPU statement; scores from
block keys stored in two stretches identical to scores from raw keys; the selection (byte mask and
position list) exact -- index work -- on random distinct scores, on ties, and at a long context;
and the whole chain scores -> select -> masked attention against the oracle's."""
import numpy as np
import pytest

from conftest import rel_l2
from gpu_util import Bufs, QwRef, NULL_REF
from qwasar_b200 import synth

pytestmark = pytest.mark.gpu


def run(be, fn):
    c = be.cmd_begin()
    fn(c)
    be.cmd_wait(c); be.cmd_free(c)


@pytest.mark.parametrize("rows,nq,d,ratio,base,max_ctx", [(5, 4, 128, 4, 13, 64), (1, 8, 128, 4, 4095, 4200), (7, 2, 64, 8, 250, 512),
                                                          (3, 4, 256, 4, 30, 64)])
def test_scores_and_pooled_scores(be, oracle, rows, nq, d, ratio, base, max_ctx):
    rng = np.random.default_rng(51 + rows)
    max_blocks = max_ctx // ratio
    qn = rng.standard_normal((rows, nq, d)).astype(np.float32)
    ik = rng.standard_normal((max_ctx, d)).astype(np.float32)
    w = synth.f32_to_bf16_bits(1.0 + 0.1 * rng.standard_normal(d).astype(np.float32))
    _, inv = oracle.rope_tables(64, 1e7)
    want, want_pool = oracle.qsa_scores(qn, ik, w, inv, rows, nq, d, ratio, base, 64, max_blocks, 1e-6)
    with Bufs(be) as B:
        qb, _ = B.shared(qn); kb, _ = B.shared(ik); wb, _ = B.shared(w); fb, _ = B.shared(inv)
        s1, v1 = B.shared_empty((rows, max_blocks), np.float32, fill=np.float32(-7.0))
        s2, v2 = B.shared_empty((rows, max_blocks), np.float32, fill=np.float32(-7.0))
        pb, pv = B.shared_empty((max_blocks, d), np.float32, fill=np.float32(0.0))
        all_blocks = (base + rows) // ratio
        run(be, lambda c: be.op_qsa_scores(c, QwRef(s1, 0), QwRef(qb, 0), QwRef(kb, 0), QwRef(wb, 0), QwRef(fb, 0), rows, nq, d, ratio,
                                           base, 64, max_blocks, 1e-6))

        def pooled(c):
            be.op_qsa_pool(c, QwRef(pb, 0), QwRef(kb, 0), QwRef(wb, 0), QwRef(fb, 0), d, ratio, 0, all_blocks // 2, 64, 1e-6)
            be.op_qsa_pool(c, QwRef(pb, 0), QwRef(kb, 0), QwRef(wb, 0), QwRef(fb, 0), d, ratio, all_blocks // 2, all_blocks, 64, 1e-6)
            be.op_qsa_scores_pooled(c, QwRef(s2, 0), QwRef(qb, 0), QwRef(pb, 0), rows, nq, d, ratio, base, max_blocks)
        run(be, pooled)
        got, got2, pool = np.array(v1), np.array(v2), np.array(pv)
    for r in range(rows):
        n = (base + r + 1) // ratio
        assert np.max(np.abs(got[r, :n] - want[r, :n])) < 1e-4           # the reference's bound, tests/test_sparse.c:418
        assert np.array_equal(got[r, :n], got2[r, :n]), "scores from stored block keys differ from scores from raw keys"
        assert np.all(got[r, n:] == -7.0) and np.all(got2[r, n:] == -7.0)  # blocks the row cannot see: left alone
    assert np.max(np.abs(pool[:all_blocks] - want_pool[:all_blocks])) < 1e-5


def check_select(be, oracle, scores, rows, ratio, base, topk, max_ctx):
    max_blocks = scores.shape[1]
    want_mask, want_list = oracle.qsa_select(scores, rows, ratio, base, topk, max_ctx)
    cap = topk * ratio + ratio
    with Bufs(be) as B:
        sb, _ = B.shared(scores)
        mb, mv = B.shared_empty((rows, max_ctx), np.uint8, fill=255)
        lb, lv = B.shared_empty((rows, 1 + cap), np.uint32, fill=0xFFFFFFF0)
        run(be, lambda c: be.op_qsa_select(c, QwRef(mb, 0), QwRef(lb, 0), QwRef(sb, 0), rows, ratio, base, topk, max_ctx, max_blocks))
        mask, lists = np.array(mv), np.array(lv)
    for r in range(rows):
        n_keys = base + r + 1
        assert np.array_equal(mask[r, :n_keys] != 0, want_mask[r, :n_keys] != 0), f"row {r}: mask differs"
        n = int(want_list[r, 0])
        assert int(lists[r, 0]) == n and np.array_equal(lists[r, 1:1 + n], want_list[r, 1:1 + n]), f"row {r}: list differs"
        assert np.all(lists[r, 1 + n:] == 0xFFFFFFF0)                      # nothing written past the count
    return lists


def test_select_random_distinct_scores(be, oracle):
    rng = np.random.default_rng(53)
    rows, ratio, base, topk, max_ctx = 5, 4, 13, 2, 64
    check_select(be, oracle, rng.standard_normal((rows, max_ctx // ratio)).astype(np.float32), rows, ratio, base, topk, max_ctx)


def test_select_ties_unselectable_and_few_blocks(be, oracle):
    rows, ratio, base, topk, max_ctx = 6, 4, 1, 3, 64
    scores = np.zeros((rows, 16), np.float32)                           # everything tied: the lowest indices win
    scores[4, :] = -3.4028235e38                                        # nothing above -FLT_MAX: only the tail
    scores[5, :2] = [np.nan, 1.0]                                       # a NaN never wins
    check_select(be, oracle, scores, rows, ratio, base, topk, max_ctx)
    # fewer complete blocks than the budget, and none at all
    check_select(be, oracle, np.ones((3, 16), np.float32), 3, 8, 0, 5, 64)


def test_select_long_context(be, oracle):
    rng = np.random.default_rng(7)
    rows, ratio, base, topk, max_ctx = 2, 4, 9001, 576, 9100
    scores = rng.standard_normal((rows, max_ctx // ratio)).astype(np.float32)
    scores[0, 100:140] = scores[0, 99]                                   # a run of equal scores inside
    check_select(be, oracle, scores, rows, ratio, base, topk, max_ctx)


@pytest.mark.parametrize("rows,ratio,base,topk", [(1, 4, 65535 * 4 + 2, 512), (3, 2, 20000, 300), (2, 4, 40000, 0), (1, 8, 70000, 20000)])
def test_select_rows_of_thousands_of_blocks(be, oracle, rows, ratio, base, topk):
    """Rows long enough for the eight-CTA cluster kernel: random scores with stretches of equal ones
    (also across the boundary between two CTAs' shares), zeros of both signs, unselectable entries; a
    budget of zero blocks; a budget larger than the number of blocks."""
    rng = np.random.default_rng(base % 1000 + rows)
    max_ctx = base + rows + 5
    nb = max_ctx // ratio
    scores = rng.standard_normal((rows, nb)).astype(np.float32)
    scores[:, 50:90] = scores[:, 49:50]
    scores[:, nb // 8 - 20: nb // 8 + 20] = 9.5                           # a tie among the very best, across a share boundary
    scores[:, 1000:1100:3] = 0.0; scores[:, 1001:1100:3] = -0.0
    scores[0, 2000:2100] = np.nan; scores[0, 2100:2200] = -3.4028235e38; scores[0, 2200:2210] = -np.inf
    check_select(be, oracle, scores, rows, ratio, base, topk, max_ctx)


@pytest.mark.parametrize("kind", ["all_zero", "mostly_zero", "two_values"])
def test_select_long_rows_of_mostly_equal_scores(be, oracle, kind):
    """The distributions a histogram pass likes least: every score equal (all zero: index heads that all came out
    negative), nine in ten equal, and two values only -- the lowest indices among the equals win."""
    rng = np.random.default_rng(7)
    rows, ratio, base, topk = 2, 4, 50000, 300
    max_ctx = base + rows + 3
    nb = max_ctx // ratio
    if kind == "all_zero":
        scores = np.zeros((rows, nb), np.float32)
    elif kind == "mostly_zero":
        scores = np.where(rng.random((rows, nb)) < 0.9, 0.0, np.abs(rng.standard_normal((rows, nb)))).astype(np.float32)
    else:
        scores = np.where(rng.random((rows, nb)) < 0.5, 1.25, 2.5).astype(np.float32)
    check_select(be, oracle, scores, rows, ratio, base, topk, max_ctx)


def test_scores_select_attend_chain(be, oracle):
    """Raw index keys -> scores -> selection -> masked attention, every stage on the device, against
    the oracle's chain fed with the device's scores (so that a last-bit difference of a score cannot
    flip a selection between the two)."""
    rng = np.random.default_rng(11)
    rows, nq, d, ratio, base, topk, qh, kvh = 4, 4, 128, 4, 700, 32, 8, 2
    max_ctx = 768; max_blocks = max_ctx // ratio; cap = topk * ratio + ratio
    qn = rng.standard_normal((rows, nq, d)).astype(np.float32); ik = rng.standard_normal((max_ctx, d)).astype(np.float32)
    q = rng.standard_normal((rows, qh, 256)).astype(np.float32)
    kc = synth.cache_bits(rng, kvh, max_ctx); vc = synth.cache_bits(rng, kvh, max_ctx)
    _, inv = oracle.rope_tables(64, 1e7)
    with Bufs(be) as B:
        qnb, _ = B.shared(qn); ikb, _ = B.shared(ik); fb, _ = B.shared(inv); qb, _ = B.shared(q)
        sb, sv = B.shared_empty((rows, max_blocks), np.float32, fill=np.float32(0.0))
        mb, _ = B.shared_empty((rows, max_ctx), np.uint8, fill=0)
        lb, lv = B.shared_empty((rows, 1 + cap), np.uint32, fill=0xFFFFFFF0)
        ob, ov = B.shared_empty((rows, qh, 256), np.float32)
        kb = B.device(kc); vb = B.device(vc)

        def chain(c):
            be.op_qsa_scores(c, QwRef(sb, 0), QwRef(qnb, 0), QwRef(ikb, 0), NULL_REF, QwRef(fb, 0), rows, nq, d, ratio, base, 64,
                             max_blocks, 1e-6)
            be.op_qsa_select(c, QwRef(mb, 0), QwRef(lb, 0), QwRef(sb, 0), rows, ratio, base, topk, max_ctx, max_blocks)
            be.op_attn_masked(c, QwRef(ob, 0), QwRef(qb, 0), QwRef(kb, 0), QwRef(vb, 0), QwRef(lb, 0), rows, qh, kvh, 256, max_ctx, base,
                              0.0625, topk, ratio)
        run(be, chain)
        scores, lists, got = np.array(sv), np.array(lv), np.array(ov)
    _, want_list = oracle.qsa_select(scores, rows, ratio, base, topk, max_ctx)
    for r in range(rows):
        n = int(want_list[r, 0])
        assert int(lists[r, 0]) == n and np.array_equal(lists[r, 1:1 + n], want_list[r, 1:1 + n])
    want = oracle.attn_masked(q, kc, vc, want_list, rows, qh, kvh, 256, max_ctx, 0.0625)
    assert rel_l2(got, want) < 5e-3          # the masked attention's tensor-op form (bf16 q and weights)


def test_long_row_stages_back_to_back_on_the_same_buffers(be, oracle):
    """Scoring and selection of a long row (the thread-block-cluster selection) launched several times in
    a row on the same score, mask and list buffers, with two different queries: each launch may
    start under the one before it, and the buffers must come out as the LAST pair leaves them."""
    rng = np.random.default_rng(77)
    rows, nq, d, ratio, base, topk = 1, 4, 128, 4, 40001, 256
    max_ctx = base + 63; max_blocks = max_ctx // ratio; cap = topk * ratio + ratio
    pool = rng.standard_normal((max_blocks, d)).astype(np.float32)
    qa = rng.standard_normal((rows, nq, d)).astype(np.float32); qb_ = rng.standard_normal((rows, nq, d)).astype(np.float32)
    with Bufs(be) as B:
        pb, _ = B.shared(pool); q1, _ = B.shared(qa); q2, _ = B.shared(qb_)
        sb, sv = B.shared_empty((rows, max_blocks), np.float32, fill=np.float32(0.0))
        mb, mv = B.shared_empty((rows, max_ctx), np.uint8, fill=255)
        lb, lv = B.shared_empty((rows, 1 + cap), np.uint32, fill=0xFFFFFFF0)

        def stages(c):
            for qx in (q1, q2, q1, q2):
                be.op_qsa_scores_pooled(c, QwRef(sb, 0), QwRef(qx, 0), QwRef(pb, 0), rows, nq, d, ratio, base, max_blocks)
                be.op_qsa_select(c, QwRef(mb, 0), QwRef(lb, 0), QwRef(sb, 0), rows, ratio, base, topk, max_ctx, max_blocks)
                be.op_qsa_select(c, QwRef(mb, 0), QwRef(lb, 0), QwRef(sb, 0), rows, ratio, base, topk, max_ctx, max_blocks)
        run(be, stages)
        scores, mask, lists = np.array(sv), np.array(mv), np.array(lv)

        def last_alone(c):
            be.op_qsa_scores_pooled(c, QwRef(sb, 0), QwRef(q2, 0), QwRef(pb, 0), rows, nq, d, ratio, base, max_blocks)
        run(be, last_alone)
        assert np.array_equal(scores, np.array(sv)), "the last scoring's output differs from the same scoring run alone"
    want_mask, want_list = oracle.qsa_select(scores, rows, ratio, base, topk, max_ctx)
    n_keys, n = base + 1, int(want_list[0, 0])
    assert np.array_equal(mask[0, :n_keys] != 0, want_mask[0, :n_keys] != 0)
    assert int(lists[0, 0]) == n and np.array_equal(lists[0, 1:1 + n], want_list[0, 1:1 + n])
