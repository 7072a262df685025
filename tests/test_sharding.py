"""Multi-rank partitioning on CPU: two gloo ranks reproduce the unsharded attention with the
oracle standing in for the kernels (same exchange pattern as the GPU path: all-gather of the
(acc, max, sum) partials, local merge)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from qwasar_b200 import sharding, synth


def test_plan_and_slices():
    assert sharding.plan(1, 4) == (1, 1, 1)
    assert sharding.plan(2, 4) == (2, 1, 1)
    assert sharding.plan(8, 4) == (4, 1, 2)
    assert sharding.plan(8, 2, seq_shards=8) == (1, 8, 1)
    assert sharding.plan(8, 2, seq_shards=4) == (2, 4, 1)
    with pytest.raises(ValueError):
        sharding.plan(8, 2, seq_shards=3)
    assert sharding.head_slice(1, 2, 24, 4) == ((12, 24), (2, 4))
    assert sharding.head_slice(3, 4, 16, 4) == ((12, 16), (3, 4))
    # ranges tile [0, n) exactly, page-aligned, trailing shards may be empty
    for n, s in ((262145, 8), (130, 4), (64, 2), (1, 8)):
        r = [sharding.seq_range(i, s, n) for i in range(s)]
        assert r[0][0] == 0 and r[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all(lo % 64 == 0 for lo, hi in r if lo < n)
        assert sharding.owner_of_position(n - 1, s, n) == max(i for i, (lo, hi) in enumerate(r) if hi > lo)
    coords = [sharding.rank_coords(r, 8, 2, seq_shards=4) for r in range(8)]
    assert coords[0] == (0, 0, 0) and coords[3] == (0, 0, 3) and coords[4] == (0, 1, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.oracle import Oracle
    orc = Oracle()
    rng = np.random.default_rng(11)                      # every rank draws the same problem
    rows, qh, kvh, base = 2, 8, 2, 300
    n_keys = base + rows
    q = synth.normal_bf16(rng, (rows, qh, 256)); gate = synth.normal_bf16(rng, (rows, qh, 256))
    kc = synth.cache_bits(rng, kvh, n_keys); vc = synth.cache_bits(rng, kvh, n_keys)
    whole = orc.mul_sigmoid(orc.attn_decode(q, kc, vc, rows, qh, kvh, 256, n_keys, base, synth.SCALE, threads=1), gate)
    if mode == "seq":
        lo, hi = sharding.seq_range(rank, world, n_keys)
        part = np.zeros((rows * qh, 258), np.float32)
        for r in range(rows):
            for h in range(qh):
                acc, st = orc.attn_partial(q[r, h], kc[h // (qh // kvh)], vc[h // (qh // kvh)], lo,
                                           min(hi, base + r + 1), 256, synth.SCALE)
                part[r * qh + h, :256] = acc; part[r * qh + h, 256:] = st
        gathered = [torch.empty(rows * qh, 258) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(part))
        g = np.stack([t.numpy() for t in gathered])
        out = np.stack([orc.attn_merge(g[:, i, :256], g[:, i, 256:], gate.reshape(-1, 256)[i])
                        for i in range(rows * qh)]).reshape(rows, qh, 256)
    else:   # kv-head sharding: no exchange inside attention; gather the head slices for the comparison
        (q0, q1), (k0, k1) = sharding.head_slice(rank, world, qh, kvh)
        mine = orc.attn_decode(np.ascontiguousarray(q[:, q0:q1]), np.ascontiguousarray(kc[k0:k1]),
                               np.ascontiguousarray(vc[k0:k1]), rows, q1 - q0, k1 - k0, 256, n_keys, base,
                               synth.SCALE, threads=1)
        mine = orc.mul_sigmoid(mine, np.ascontiguousarray(gate[:, q0:q1]))
        gathered = [torch.empty(rows, q1 - q0, 256) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(mine))
        out = np.concatenate([t.numpy() for t in gathered], axis=1)
    err = float(np.abs(out - whole).max() / np.abs(whole).max())
    out_q.put((rank, err, bool(np.array_equal(out, whole))))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["seq", "heads"])
def test_two_ranks_reproduce_the_whole(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, exact in res:
        if mode == "heads":
            assert exact, f"rank {rank}: head sharding must be bit-identical"
        else:
            assert err < 1e-6, f"rank {rank}: merged partials differ by {err}"
