"""Seeded synthetic workloads for the attention path, shared by the benchmark,
the smoke check and the tests.  The shapes are the reference's (Qwen3.5-9B,
Qwen3.8-27B, a Flash-Next-like dense grouping); the values are bf16-exact
N(0,1) draws, as no dataset or checkpoint is involved anywhere on this path
(the reference's own attention benches fill synthetic caches too,
tools/bench/attnbench.c:24-26)."""
from __future__ import annotations

import numpy as np

HEAD_DIM = 256
ROTARY_DIM = 64
ROPE_THETA = 1e7
MROPE_SECTION = (11, 11, 10)
EPS = 1e-6
SCALE = 1.0 / 16.0      # 1 / sqrt(256)

# name -> geometry.  `base_pos` keys are already cached; `rows` new tokens arrive.
WORKLOADS = {
    "c1_9b_decode_4k":     dict(q_heads=16, kv_heads=4, rows=1, base_pos=4096, batch=(1,), seed=0, layers=8),
    "c2_9b_prefill_4k":    dict(q_heads=16, kv_heads=4, rows=4096, base_pos=0, batch=(1,), seed=1, layers=8),
    "c3_27b_decode_32k":   dict(q_heads=24, kv_heads=4, rows=1, base_pos=32768, batch=(1, 8), seed=2, layers=16),
    "c4_27b_verify_32k":   dict(q_heads=24, kv_heads=4, rows=4, base_pos=32768, batch=(1,), seed=3, layers=16),
    "c5_flash_decode_262k": dict(q_heads=16, kv_heads=2, rows=1, base_pos=262144, batch=(1, 4), seed=4, layers=12),
}


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (finite input)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + r) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 values that are exactly representable in bf16."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def normal_bf16(rng, shape) -> np.ndarray:
    """N(0,1) draws rounded to bf16, returned widened to float32."""
    return bf16_round(rng.standard_normal(shape, dtype=np.float32))


def positions(base_pos: int, rows: int) -> np.ndarray:
    """Text positions: the three MRoPE axes agree (qwasar_graph.c:1540-1547)."""
    return np.tile(np.arange(base_pos, base_pos + rows, dtype=np.int32), (3, 1))


def rope_tables(rotary_dim=ROTARY_DIM, theta=ROPE_THETA, section=MROPE_SECTION):
    """axis / inv_freq exactly as qw_rope_tables computes them in fp32
    (qwasar_cpu.c:284-302): numpy float32 powf is not guaranteed bit-identical
    to libm, so callers that need the reference's bits take the tables from the
    backend's or the oracle's qw_rope_tables instead."""
    half = rotary_dim // 2
    axis = np.zeros(half, np.uint8)
    for d in (1, 2):
        lim = min(section[d] * 3, half)
        axis[d:lim:3] = d
    j = np.arange(half, dtype=np.float32)
    inv = (np.float32(1.0) / np.power(np.float32(theta), (2 * j) / np.float32(rotary_dim), dtype=np.float32))
    return axis, inv.astype(np.float32)


def step_inputs(rng, rows, q_heads, kv_heads):
    """One step's activations: qg [rows, q_heads, 512], k and v [rows, kv_heads, 256]."""
    qg = normal_bf16(rng, (rows, q_heads, 2 * HEAD_DIM))
    k = normal_bf16(rng, (rows, kv_heads, HEAD_DIM))
    v = normal_bf16(rng, (rows, kv_heads, HEAD_DIM))
    return qg, k, v


def cache_bits(rng, kv_heads, n_tokens) -> np.ndarray:
    """bf16 bit patterns of an N(0,1) cache prefix [kv_heads, n_tokens, 256]."""
    return f32_to_bf16_bits(rng.standard_normal((kv_heads, n_tokens, HEAD_DIM), dtype=np.float32))


def decode_kv_bytes(n_keys: int, kv_heads: int) -> int:
    """Unique K+V bytes one sequence's attention reads per layer
    (tools/bench/attnbench.c:45)."""
    return n_keys * kv_heads * HEAD_DIM * 2 * 2


def prefill_flops(rows: int, base_pos: int, q_heads: int) -> float:
    """4 * q_heads * head_dim * sum_r (base_pos + r + 1): the causal count, in the
    convention of tools/bench/fabench.c:37-38."""
    keys = rows * base_pos + rows * (rows + 1) / 2
    return 4.0 * q_heads * HEAD_DIM * keys
