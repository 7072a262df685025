"""Host logic of the split-KV decode kernel: how a launch's (sequence, kv head) groups, laid end to
end as one line of 32-key tiles, are cut into one share per CTA.  No GPU needed: the library's own
arithmetic (the function the kernel and the host's merge decision share) through qw_attn_split_plan."""
import ctypes as C

import numpy as np
import pytest

import qwasar_b200

SEG_COST = 3


def plan(lib, n_keys, kv_heads, n_cta_max=148):
    keys = np.asarray(n_keys, np.int32)
    shares = np.zeros(n_cta_max + 1, np.int32)
    merge = C.c_int32(-1)
    n = lib.qw_attn_split_plan(len(keys), kv_heads, keys.ctypes.data, n_cta_max, shares.ctypes.data, C.addressof(merge))
    return n, shares[:n + 1].astype(np.int64), merge.value


@pytest.fixture(scope="module")
def lib():
    return qwasar_b200.load_library()


def group_ranges(n_keys, kv_heads):
    out, cum = [], 0
    for k in n_keys:
        t = (k + 31) // 32
        for _ in range(kv_heads):
            out.append((cum, cum + t)); cum += t
    return out, cum


@pytest.mark.parametrize("n_keys,kv_heads", [([32769] * 8, 4), ([32769], 4), ([262145], 2), ([4097], 4), ([1], 1),
                                             ([5, 70, 3000, 64], 2), ([33] * 16, 8), ([100000, 10], 1)])
def test_shares_cover_the_line_in_order(lib, n_keys, kv_heads):
    n, shares, merge = plan(lib, n_keys, kv_heads)
    groups, total = group_ranges(n_keys, kv_heads)
    assert n == min(148, total)
    assert shares[0] == 0 and shares[-1] == total
    assert np.all(np.diff(shares) >= 0)
    # the merge is needed exactly when some group meets more than one non-empty share
    cut = any(sum(1 for c in range(n) if shares[c] < g1 and shares[c + 1] > g0) > 1 for g0, g1 in groups)
    assert merge == int(cut)


def test_shares_are_equal_in_cost_not_in_tiles(lib):
    """Headline shape: 8 sequences x 4 heads x 1025 tiles over 148 CTAs.  A share that begins a group
    is shorter by the cost of a segment start (3 tiles), all costs within one tile of each other."""
    n_keys, kv_heads = [32769] * 8, 4
    n, shares, _ = plan(lib, n_keys, kv_heads)
    groups, total = group_ranges(n_keys, kv_heads)
    starts = {g0 for g0, _ in groups}
    cost = []
    for c in range(n):
        inside = sum(1 for g0 in starts if shares[c] <= g0 < shares[c + 1])
        cost.append((shares[c + 1] - shares[c]) + SEG_COST * inside)
    assert max(cost) - min(cost) <= SEG_COST + 1
    assert abs(np.mean(cost) - (total + SEG_COST * len(groups)) / n) < 1e-6


def test_random_shapes(lib):
    rng = np.random.default_rng(0)
    for _ in range(300):
        n_seq = int(rng.integers(1, 17)); kv_heads = int(rng.choice([1, 2, 4, 8]))
        n_keys = [int(rng.choice([1, 31, 32, 33, 100, 2049, 40000])) if rng.random() < 0.6 else int(rng.integers(1, 90000))
                  for _ in range(n_seq)]
        n, shares, merge = plan(lib, n_keys, kv_heads, n_cta_max=int(rng.choice([1, 4, 148, 200])))
        groups, total = group_ranges(n_keys, kv_heads)
        assert shares[0] == 0 and shares[-1] == total and np.all(np.diff(shares) >= 0)
        for g0, g1 in groups:                                  # the CTAs of a group are consecutive
            hit = [c for c in range(n) if shares[c] < g1 and shares[c + 1] > g0]
            assert hit == list(range(hit[0], hit[-1] + 1))


def test_bad_arguments(lib):
    shares = np.zeros(149, np.int32)
    keys = np.asarray([0], np.int32)
    assert lib.qw_attn_split_plan(1, 4, keys.ctypes.data, 148, shares.ctypes.data, None) == 0
    assert lib.qw_attn_split_plan(0, 4, keys.ctypes.data, 148, shares.ctypes.data, None) == 0
    assert lib.qw_attn_split_plan(1, 4, None, 148, shares.ctypes.data, None) == 0
