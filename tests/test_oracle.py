"""The CPU oracle against everything that pins it: the reference's known answers,
the fixtures its own compiled code produced, and (where oracle/_ref is present)
that compiled code itself, bit for bit."""
import os
import sys

import numpy as np
import pytest

from conftest import rel_l2, xorshift_fill
from oracle.oracle import BF16, F16
from qwasar_b200 import synth

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden  # noqa: E402

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "attn_golden.npz"))


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_rope_tables_known_answers(oracle):
    """tests/test_ops.c:163-182: axis pattern 0,1,2,... ending 0,1; counts 11/11/10;
    inv_freq[0,1,2,31] for (64, 1e7)."""
    axis, inv = oracle.rope_tables(64, 1e7, (11, 11, 10))
    expect = [0, 1, 2] * 10 + [0, 1]
    assert axis.tolist() == expect
    assert [int((axis == a).sum()) for a in range(3)] == [11, 11, 10]
    assert abs(inv[0] - 1.0) < 1e-9
    assert abs(inv[1] - 0.6042963862) < 1e-7
    assert abs(inv[2] - 0.3651741147) < 1e-7
    assert abs(inv[31] - 1.654816941254e-07) < 1e-13
    assert np.array_equal(axis, GOLDEN["rope_axis"])
    assert np.array_equal(bits(inv), bits(GOLDEN["rope_inv_freq"]))


def test_synth_tables_match(oracle):
    axis, inv = oracle.rope_tables()
    a2, i2 = synth.rope_tables()
    assert np.array_equal(axis, a2)
    np.testing.assert_allclose(inv, i2, rtol=1e-6)


def test_cache_conversions(oracle):
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(200000).astype(np.float32) * 10,
                        np.float32([0.0, -0.0, 1.0, 30.0, -999.0, 1e-30, 3.3895e38, 65504.0])])
    assert np.array_equal(oracle.to_cache(x, BF16), synth.f32_to_bf16_bits(x))
    assert np.array_equal(bits(oracle.from_cache(oracle.to_cache(x, BF16), BF16)), bits(synth.bf16_round(x)))
    fin = np.abs(x) < 6e4
    assert np.array_equal(oracle.to_cache(x[fin], F16), x[fin].astype(np.float16).view(np.uint16))
    # the two encodings of 1.0 the reference source yields under its two builds
    assert int(oracle.to_cache(np.float32([1.0]), BF16)[0]) == 0x3F80
    assert int(oracle.to_cache(np.float32([1.0]), F16)[0]) == 0x3C00


@pytest.mark.parametrize("case", make_golden.CASES, ids=[c[0] for c in make_golden.CASES])
def test_golden_fixture(oracle, case):
    """The restatement reproduces, bit for bit, what the reference's compiled CPU
    code produced for the committed cases (inputs regenerated from the seed)."""
    name, rows, qh, kvh, base, ctx, seed, mm = case
    qg, k, v, kc, vc, pos, w = make_golden.case_inputs(rows, qh, kvh, base, ctx, seed, mm, name)
    want_sha = bytes(GOLDEN[name + "/input_sha256"]).hex()
    assert make_golden.digest(qg, k, v, kc, vc, pos, w) == want_sha, "input generator drifted"
    axis, inv = oracle.rope_tables()
    kcb, vcb = kc.copy(), vc.copy()
    out, q_post, k_post = oracle.attn_layer(qg, k, v, w, w, pos, axis, inv, kcb, vcb, rows, qh, kvh, 256, 64, ctx,
                                            base, 1e-6, 0.0625, BF16, threads=1, want_post=True)
    assert np.array_equal(bits(q_post), bits(GOLDEN[name + "/q_post"]))
    assert np.array_equal(bits(k_post), bits(GOLDEN[name + "/k_post"]))
    assert np.array_equal(kcb[:, base:base + rows], GOLDEN[name + "/kc_rows"])
    assert np.array_equal(vcb[:, base:base + rows], GOLDEN[name + "/vc_rows"])
    # untouched slots stay untouched
    assert np.array_equal(kcb[:, :base], kc[:, :base]) and np.array_equal(kcb[:, base + rows:], kc[:, base + rows:])
    gate = np.ascontiguousarray(qg.reshape(rows, qh, 512)[:, :, 256:])
    want = oracle.mul_sigmoid(GOLDEN[name + "/attn_pre_gate"], gate)
    assert np.array_equal(bits(out), bits(want))
    # the shipped half-precision cache, same inputs
    kch = oracle.to_cache(oracle.from_cache(kc, BF16), F16)
    vch = oracle.to_cache(oracle.from_cache(vc, BF16), F16)
    out_h = oracle.attn_layer(qg, k, v, w, w, pos, axis, inv, kch, vch, rows, qh, kvh, 256, 64, ctx, base, 1e-6,
                              0.0625, F16, threads=1)
    want_h = oracle.mul_sigmoid(GOLDEN[name + "/attn_pre_gate_f16"], gate)
    assert np.array_equal(bits(out_h), bits(want_h))
    # bf16 vs half cache: same function, different rounding of K/V only
    assert rel_l2(out, out_h) < 2e-2


def test_against_compiled_reference(oracle, refcpu):
    """Random shapes: every stage equal to the reference's compiled functions, bitwise."""
    rng = np.random.default_rng(77)
    axis, inv = refcpu.rope_tables()
    for _ in range(6):
        rows = int(rng.integers(1, 6)); kvh = int(rng.integers(1, 4)); gqa = int(rng.choice([1, 4, 6, 8]))
        qh = kvh * gqa; base = int(rng.integers(0, 150)); ctx = base + rows + int(rng.integers(0, 9))
        qg, k, v = synth.step_inputs(rng, rows, qh, kvh)
        kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
        pos = synth.positions(base, rows)
        pos[1] += int(rng.integers(0, 50)); pos[2] += int(rng.integers(0, 50))
        w = synth.f32_to_bf16_bits(rng.standard_normal(256).astype(np.float32))
        k1, v1, k2, v2 = kc.copy(), vc.copy(), kc.copy(), vc.copy()
        out, qp, kp = oracle.attn_layer(qg, k, v, w, None, pos, axis, inv, k1, v1, rows, qh, kvh, 256, 64, ctx, base,
                                        1e-6, 0.0625, BF16, threads=2, want_post=True)
        pre, gate, qp2, kp2 = refcpu.attn_layer(qg, k, v, w, None, pos, axis, inv, k2, v2, rows, qh, kvh, 256, 64,
                                                ctx, base, 1e-6, 0.0625, threads=1)
        assert np.array_equal(bits(qp), bits(qp2)) and np.array_equal(bits(kp), bits(kp2))
        assert np.array_equal(k1, k2) and np.array_equal(v1, v2)
        assert np.array_equal(bits(out), bits(oracle.mul_sigmoid(pre, gate)))


def test_reference_test_generator_and_shape(oracle, refcpu):
    """One shape of the reference's own attention test (tests/test_attn.c:56-141) with its
    xorshift inputs: cache primed through kv_write, tail poisoned, attention compared."""
    qh, kvh, hd, ctx, base, rows = 24, 4, 256, 96, 50, 4
    hk = xorshift_fill(base * kvh * hd, 0x5150).reshape(base, kvh, hd)
    hv = xorshift_fill(base * kvh * hd, 0x6161).reshape(base, kvh, hd)
    kc = np.zeros((kvh, ctx, hd), np.uint16); vc = np.zeros((kvh, ctx, hd), np.uint16)
    oracle.kv_write(kc, vc, hk, hv, base, kvh, hd, ctx, 0)
    kc[:, base + rows:] = oracle.to_cache(np.float32([30.0]))[0]
    vc[:, base + rows:] = oracle.to_cache(np.float32([-999.0]))[0]
    q = xorshift_fill(rows * qh * hd, 0x1717).reshape(rows, qh, hd)
    k = xorshift_fill(rows * kvh * hd, 0x2727).reshape(rows, kvh, hd)
    v = xorshift_fill(rows * kvh * hd, 0x3737).reshape(rows, kvh, hd)
    k2, v2 = kc.copy(), vc.copy()
    oracle.kv_write(kc, vc, k, v, rows, kvh, hd, ctx, base)
    refcpu.kv_write(k2, v2, k, v, rows, kvh, hd, ctx, base)
    assert np.array_equal(kc, k2) and np.array_equal(vc, v2)
    a = oracle.attn_decode(q, kc, vc, rows, qh, kvh, hd, ctx, base, 0.0625, threads=1)
    b = refcpu.attn_decode(q, kc, vc, rows, qh, kvh, hd, ctx, base, 0.0625, threads=1)
    c = refcpu.attn_decode(q, kc, vc, rows, qh, kvh, hd, ctx, base, 0.0625, threads=4)   # sliced driver
    assert np.array_equal(bits(a), bits(b)) and np.array_equal(bits(b), bits(c))
    assert np.abs(a).max() < 1.5          # a kernel that read the poison would be near -999


def test_gqa_and_normalisation(oracle):
    """tests/test_attn.c:199-238: V constant per kv head => output = h / gqa + 1."""
    qh, kvh, hd, ctx, n = 24, 4, 256, 64, 33
    rng = np.random.default_rng(3)
    q = rng.standard_normal((1, qh, hd)).astype(np.float32)
    kc = np.zeros((kvh, ctx, hd), np.uint16)
    vc = np.zeros((kvh, ctx, hd), np.uint16)
    for h in range(kvh):
        vc[h, :n] = oracle.to_cache(np.float32([h + 1.0]))[0]
    out = oracle.attn_decode(q, kc, vc, 1, qh, kvh, hd, ctx, n - 1, 0.0625)
    want = (np.arange(qh) // (qh // kvh) + 1).astype(np.float32)
    assert np.abs(out[0] - want[:, None]).max() < 1e-4


def test_causality(oracle):
    """tests/test_attn.c:148-194: poisoning keys past the query's position changes nothing."""
    qh, kvh, hd, ctx, base = 8, 2, 256, 128, 40
    rng = np.random.default_rng(4)
    q = rng.standard_normal((1, qh, hd)).astype(np.float32)
    kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
    a = oracle.attn_decode(q, kc, vc, 1, qh, kvh, hd, ctx, base, 0.0625)
    kc[:, base + 1:] = oracle.to_cache(np.float32([50.0]))[0]
    vc[:, base + 1:] = oracle.to_cache(np.float32([-999.0]))[0]
    b = oracle.attn_decode(q, kc, vc, 1, qh, kvh, hd, ctx, base, 0.0625)
    assert np.array_equal(bits(a), bits(b))


def test_partials_merge_to_whole(oracle):
    """Splitting the keys anywhere and merging by log-sum-exp (metal/attn.metal:273-331)
    gives the unsplit attention; empty parts drop out; the gate applies once."""
    hd, n = 256, 300
    rng = np.random.default_rng(9)
    q = rng.standard_normal(hd).astype(np.float32)
    kh = synth.cache_bits(rng, 1, n)[0]; vh = synth.cache_bits(rng, 1, n)[0]
    gate = rng.standard_normal(hd).astype(np.float32)
    whole = oracle.attn_decode(q.reshape(1, 1, hd), kh.reshape(1, n, hd), vh.reshape(1, n, hd), 1, 1, 1, hd, n, n - 1,
                               0.0625)[0, 0]
    for cuts in ([0, 300], [0, 64, 300], [0, 1, 2, 128, 128, 299, 300], [0, 0, 300, 300]):
        parts = [oracle.attn_partial(q, kh, vh, a, b, hd, 0.0625) for a, b in zip(cuts[:-1], cuts[1:])]
        pacc = np.stack([p[0] for p in parts]); pstat = np.stack([p[1] for p in parts])
        got = oracle.attn_merge(pacc, pstat)
        assert rel_l2(got, whole) < 1e-6
        gated = oracle.attn_merge(pacc, pstat, gate)
        assert rel_l2(gated, oracle.mul_sigmoid(whole, gate)) < 1e-6
    # nothing live at all -> zeros, not NaN
    z = oracle.attn_merge(np.zeros((3, hd), np.float32), np.zeros((3, 2), np.float32))
    assert np.array_equal(z, np.zeros(hd, np.float32))


def test_fast_math_build_is_immaterial(oracle):
    """The timed build uses the reference's -O3 -ffast-math; the truth build is strict.
    They agree far inside every tolerance used anywhere."""
    from oracle.oracle import Oracle
    fast = Oracle(fast=True)
    rng = np.random.default_rng(21)
    rows, qh, kvh, ctx, base = 2, 8, 2, 600, 500
    q = rng.standard_normal((rows, qh, 256)).astype(np.float32)
    kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
    a = oracle.attn_decode(q, kc, vc, rows, qh, kvh, 256, ctx, base, 0.0625)
    b = fast.attn_decode(q, kc, vc, rows, qh, kvh, 256, ctx, base, 0.0625)
    assert rel_l2(b, a) < 1e-5


def test_masked_attention_is_the_reference_function_over_the_listed_rows(oracle, refcpu):
    """orc_attn_masked (attention over a list of visible positions, qwasar_gpu.h:635-645) against the
    reference's own compiled qw_cpu_attn_decode: over the K/V rows of the list gathered into a dense
    cache of that many positions the two are the same arithmetic in the same order -- bit for bit."""
    rng = np.random.default_rng(42)
    rows, qh, kvh, ctx, cap = 5, 12, 2, 700, 96
    q = rng.standard_normal((rows, qh, 256)).astype(np.float32)
    kc = synth.cache_bits(rng, kvh, ctx); vc = synth.cache_bits(rng, kvh, ctx)
    lists = np.full((rows, 1 + cap), 0xFFFFFFF0, np.uint32)             # poisoned past the count
    for r in range(rows):
        n = [1, 3, cap, 17, cap - 1][r]
        lists[r, 0] = n
        lists[r, 1:1 + n] = np.sort(rng.choice(ctx, n, replace=False))
    got = oracle.attn_masked(q, kc, vc, lists, rows, qh, kvh, 256, ctx, 0.0625)
    for r in range(rows):
        n = int(lists[r, 0]); pos = lists[r, 1:1 + n].astype(np.int64)
        want = refcpu.attn_decode(q[r:r + 1], np.ascontiguousarray(kc[:, pos]), np.ascontiguousarray(vc[:, pos]),
                                  1, qh, kvh, 256, n, n - 1, 0.0625)
        assert np.array_equal(got[r], want[0])


def test_qsa_scores_are_the_reference_functions_composed(oracle, refcpu):
    """orc_qsa_scores against the composition the reference's own test writes out
    (tests/test_sparse.c:392-416) from its compiled qw_cpu_rms_norm and qw_cpu_rope_partial:
    bit for bit, block keys and scores."""
    rng = np.random.default_rng(51)
    rows, nq, d, ratio, base, max_ctx, rd = 5, 4, 128, 4, 13, 64, 64
    max_blocks = max_ctx // ratio
    qn = rng.standard_normal((rows, nq, d)).astype(np.float32)
    ik = rng.standard_normal((max_ctx, d)).astype(np.float32)
    w = synth.f32_to_bf16_bits(1.0 + 0.1 * rng.standard_normal(d).astype(np.float32))
    axis, inv = refcpu.rope_tables(rd, 1e7)
    got, pool = oracle.qsa_scores(qn, ik, w, inv, rows, nq, d, ratio, base, rd, max_blocks, 1e-6)
    for r in range(rows):
        n_blocks = (base + r + 1) // ratio
        assert np.all(np.isnan(got[r, n_blocks:]))
        for b in range(n_blocks):
            pooled = np.zeros(d, np.float32)
            for t in range(ratio):
                pooled = pooled + ik[b * ratio + t]
            pooled = pooled / np.float32(ratio)
            kn = refcpu.rms_norm(pooled[None], w, d, 1, 1e-6)
            kn = refcpu.rope_partial(kn, np.full((3, 1), b * ratio, np.int32), axis, inv, 1, 1, d, rd)[0]
            assert np.array_equal(kn, pool[b])
            s = np.float32(0)
            for h in range(nq):
                dot = np.float32(0)
                for i in range(d):
                    dot = np.float32(dot + qn[r, h, i] * kn[i])
                if dot > 0:
                    s = np.float32(s + dot)
            assert got[r, b] == np.float32(s / np.float32(np.sqrt(np.float32(d))))


def test_qsa_select_known_answers(oracle):
    """Top-k blocks by repeated arg-max (lowest index among equals), the trailing incomplete block
    always visible, the list = the mask's positions ascending (qwasar_flash_cpu.c:363-406)."""
    ratio, base, topk, max_ctx = 4, 13, 2, 64
    scores = np.zeros((3, 16), np.float32)
    scores[0, :3] = [0.5, 0.9, 0.1]          # 14 keys: 3 blocks + tail {12, 13}
    scores[1, :3] = [0.7, 0.7, 0.7]          # 15 keys: ties -> blocks 0 and 1
    scores[2, :4] = [0.1, -3.0e38, 0.3, 0.2]  # 16 keys: 4 blocks, no tail
    mask, lists = oracle.qsa_select(scores, 3, ratio, base, topk, max_ctx)
    vis = lambda r: list(np.nonzero(mask[r, :base + r + 1] == 1)[0])
    assert vis(0) == [0, 1, 2, 3, 4, 5, 6, 7, 12, 13]
    assert vis(1) == [0, 1, 2, 3, 4, 5, 6, 7, 12, 13, 14]
    assert vis(2) == [8, 9, 10, 11, 12, 13, 14, 15]
    for r in range(3):
        assert np.all(mask[r, base + r + 1:] == 255)                     # positions the row cannot see: not written
        n = int(lists[r, 0])
        assert list(lists[r, 1:1 + n]) == vis(r)


def q4_weights(rng, n, k, group):
    """MLX affine 4-bit: U32 [n, k/8] nibbles, bf16 scales (both signs) and biases [n, k/group]."""
    w = rng.integers(0, 2 ** 32, (n, k // 8), dtype=np.uint64).astype(np.uint32)
    sc = synth.f32_to_bf16_bits((0.02 * rng.standard_normal((n, k // group))).astype(np.float32))
    bi = synth.f32_to_bf16_bits((0.1 * rng.standard_normal((n, k // group))).astype(np.float32))
    return w, sc, bi


@pytest.mark.parametrize("k,n,rows,group", [(64, 3, 1, 64), (512, 48, 2, 64), (256, 5, 3, 32), (1024, 17, 1, 32)])
def test_q4_product_is_the_reference_function(oracle, refcpu, k, n, rows, group):
    """orc_qmv_q4 against the compiled qw_cpu_qmv_q4 (qwasar_cpu.c:36-63): bit for bit."""
    rng = np.random.default_rng(k + n)
    w, sc, bi = q4_weights(rng, n, k, group)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    assert np.array_equal(oracle.qmv_q4(x, w, sc, bi, k, n, rows, group), refcpu.qmv_q4(x, w, sc, bi, k, n, rows, group))


# ---- the reference's own block selection and composed layer (qwasar_flash_cpu.c) ------------------
def _q4(rng, n, k, group=64, scale=0.02):
    w = rng.integers(0, 2 ** 32, (n, k // 8), dtype=np.uint64).astype(np.uint32)
    sc = synth.f32_to_bf16_bits((scale * rng.standard_normal((n, k // group))).astype(np.float32))
    bi = synth.f32_to_bf16_bits((-7.5 * scale * (1 + 0.1 * rng.standard_normal((n, k // group)))).astype(np.float32))
    return w, sc, bi


def _identity_q4(n, group=64):
    """A 4-bit affine matrix that is exactly the identity: nibble 1 on the diagonal, scale 1, bias 0."""
    w = np.zeros((n, n // 8), np.uint32)
    for i in range(n):
        w[i, i // 8] = np.uint32(1) << np.uint32(4 * (i % 8))
    return w, np.full((n, n // group), 0x3F80, np.uint16), np.zeros((n, n // group), np.uint16)


def _flash_layer(rng, *, q_heads, kv_heads, idx_heads, idx_dim, budget, ratio, max_ctx, hidden=256):
    from oracle.oracle import RefFlash
    if not RefFlash.available():
        pytest.skip("oracle/_ref/libqwflashcpu.so not built (needs the reference checkout at build time)")
    norm = lambda n: synth.f32_to_bf16_bits((1.0 + 0.2 * rng.standard_normal(n)).astype(np.float32))
    proj = {"q_proj": _q4(rng, q_heads * 512, hidden), "k_proj": _q4(rng, kv_heads * 256, hidden),
            "v_proj": _q4(rng, kv_heads * 256, hidden), "o_proj": _identity_q4(q_heads * 256),
            "qk_proj": _q4(rng, (idx_heads + 1) * idx_dim, hidden)}
    norms = {"q_norm": norm(256), "k_norm": norm(256), "idx_q_norm": norm(idx_dim), "idx_k_norm": norm(idx_dim)}
    fl = RefFlash(hidden=hidden, hidden_out=q_heads * 256, q_heads=q_heads, kv_heads=kv_heads, head_dim=256, idx_heads=idx_heads,
                  idx_dim=idx_dim, budget=budget, ratio=ratio, max_ctx=max_ctx, proj=proj, norms=norms)
    return fl, norms


@pytest.mark.parametrize("ratio,topk,idx_dim", [(4, 3, 128), (2, 5, 64), (8, 2, 128)])
def test_qsa_select_is_the_reference_function(oracle, refcpu, ratio, topk, idx_dim):
    """orc_qsa_scores + orc_qsa_select against the reference's own qsa_select, token by token over a
    growing context: the same mask of visible positions at every step.  The reference's selection is
    a repeated arg-max with the lowest index among equals; blocks whose heads all score <= 0 tie at
    exactly 0, and the last tokens here are zero vectors, which ties every block."""
    rng = np.random.default_rng(ratio * 100 + topk)
    nq, P, hidden = 4, 70, 256
    fl, norms = _flash_layer(rng, q_heads=2, kv_heads=1, idx_heads=nq, idx_dim=idx_dim, budget=topk * ratio, ratio=ratio, max_ctx=P)
    axis, inv = refcpu.rope_tables(64, 1e7, (11, 11, 10))
    ikeys = np.zeros((P, idx_dim), np.float32)
    ties = 0
    for pos in range(P):
        x = rng.standard_normal(hidden).astype(np.float32) if pos < P - 6 else np.zeros(hidden, np.float32)
        allowed, qk = fl.select(x, pos)
        ikeys[pos] = qk[nq * idx_dim:]
        qn = refcpu.rms_norm(qk[:nq * idx_dim].reshape(nq, idx_dim), norms["idx_q_norm"], idx_dim, nq, 1e-6)
        qn = refcpu.rope_partial(qn, np.full((3, 1), pos, np.int32), axis, inv, 1, nq, idx_dim, 64)
        max_blocks = (P + ratio - 1) // ratio
        scores, _ = oracle.qsa_scores(qn, ikeys[:pos + 1], norms["idx_k_norm"], inv, 1, nq, idx_dim, ratio, pos, 64, max_blocks, 1e-6)
        mask, lists = oracle.qsa_select(scores, 1, ratio, pos, topk, P)
        assert np.array_equal(mask[0, :pos + 1], allowed), f"position {pos}"
        n_blocks = (pos + 1) // ratio
        ties += int(n_blocks > topk and len(np.unique(scores[0, :n_blocks])) < n_blocks)
        cnt = int(lists[0, 0])
        assert np.array_equal(lists[0, 1:1 + cnt], np.flatnonzero(allowed))
    assert ties > 3, "the case was meant to contain tied block scores"
    fl.close()


def test_attn_layer_is_the_reference_composition(oracle):
    """orc_attn_layer against the reference's own composed gated-attention layer, qsa_step, one token
    at a time (its cached path): projections -> split [q|gate] -> norms -> RoPE -> append -> attention
    over every position (the budget covers them all) -> sigmoid gate, read through an identity o_proj.
    qsa_step keeps its K/V cache in fp32 where this build rounds to bf16, hence a tolerance."""
    rng = np.random.default_rng(31)
    qh, kvh, P, hidden = 4, 2, 40, 256
    fl, norms = _flash_layer(rng, q_heads=qh, kv_heads=kvh, idx_heads=2, idx_dim=64, budget=4096, ratio=4, max_ctx=P)
    axis, inv = oracle.rope_tables()
    kc = np.zeros((kvh, P, 256), np.uint16); vc = np.zeros((kvh, P, 256), np.uint16)
    worst = 0.0
    for pos in range(P):
        x = rng.standard_normal(hidden).astype(np.float32)
        out, qg, k, v = fl.step(x, pos)
        got = oracle.attn_layer(qg[None], k[None], v[None], norms["q_norm"], norms["k_norm"], np.full((3, 1), pos, np.int32), axis, inv,
                                kc, vc, 1, qh, kvh, 256, 64, P, pos, 1e-6, 0.0625)
        want = out.reshape(1, qh, 256)
        err = np.sqrt(np.sum((got - want) ** 2) / np.sum(want ** 2))
        worst = max(worst, float(err))
    assert worst < 4e-3, worst
    fl.close()
