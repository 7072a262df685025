"""Host-side partitioning of the attention path over GPUs (one process per GPU).

Two shardings exist, both exact:

* KV heads: query head h reads only kv head h // gqa (qwasar_cpu.c:366), so a rank that owns
  kv heads [k0, k1) owns query heads [k0*gqa, k1*gqa) and needs nothing from the others.
* Sequence: softmax partials over disjoint key ranges combine by log-sum-exp
  (metal/attn.metal:273-331), so ranks own contiguous position ranges, exchange
  (acc, max, sum) once, and merge locally.
"""
from __future__ import annotations


def plan(world: int, kv_heads: int, seq_shards: int = 1):
    """(head_shards, seq_shards, replicas) for `world` ranks."""
    if seq_shards < 1 or world % seq_shards:
        raise ValueError("seq_shards must divide the number of ranks")
    rest = world // seq_shards
    hs = min(rest, kv_heads)
    while kv_heads % hs or rest % hs:
        hs -= 1
    return hs, seq_shards, rest // hs


def rank_coords(rank: int, world: int, kv_heads: int, seq_shards: int = 1):
    """(replica, head_shard, seq_shard) of a rank; sequence shards are the fastest-varying so that
    the ranks of one all-gather group are neighbours."""
    hs, ss, reps = plan(world, kv_heads, seq_shards)
    return rank // (hs * ss), (rank // ss) % hs, rank % ss


def head_slice(head_shard: int, head_shards: int, q_heads: int, kv_heads: int):
    """((q0, q1), (k0, k1)): the query and kv heads a head shard owns."""
    if kv_heads % head_shards or q_heads % kv_heads:
        raise ValueError("heads do not divide")
    gqa = q_heads // kv_heads
    per = kv_heads // head_shards
    k0, k1 = head_shard * per, (head_shard + 1) * per
    return (k0 * gqa, k1 * gqa), (k0, k1)


def seq_range(seq_shard: int, seq_shards: int, n_keys: int, align: int = 64):
    """[lo, hi): the key positions a sequence shard owns; boundaries are page-aligned
    (qw_op_attn_partial wants key_lo to be a multiple of 64).  Trailing shards may be empty."""
    span = -(-n_keys // seq_shards)
    span = -(-span // align) * align
    lo = min(n_keys, seq_shard * span)
    hi = min(n_keys, (seq_shard + 1) * span)
    return lo, hi


def owner_of_position(pos: int, seq_shards: int, n_keys: int, align: int = 64) -> int:
    """The sequence shard that appends the token at `pos`."""
    for s in range(seq_shards):
        lo, hi = seq_range(s, seq_shards, n_keys, align)
        if lo <= pos < hi:
            return s
    return seq_shards - 1
