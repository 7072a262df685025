"""Generates tests/golden/attn_golden.npz from the reference's own CPU code.

Run in a container that has the reference checkout (oracle/Makefile then builds
oracle/_ref/ from the reference's unmodified qwasar_cpu.c):

    make -C oracle && python tests/golden/make_golden.py

Each case's inputs are regenerated from its seed by `case_inputs` below (the
fixture stores a SHA-256 of the input bytes so that a change in the generator
is told apart from a change in the arithmetic); the stored outputs are what
qw_cpu_rms_norm / qw_cpu_rope_partial / qw_cpu_kv_write / qw_cpu_attn_decode
produced, composed in the order of qwasar_graph.c:630-659, with the cache
element type bf16 (-D__fp16=__bf16) and, for the same inputs, IEEE half."""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from qwasar_b200 import synth  # noqa: E402

# (name, rows, q_heads, kv_heads, base_pos, max_ctx, seed, multimodal positions)
CASES = [
    ("first_token", 1, 8, 2, 0, 16, 11, False),
    ("one_prior", 1, 8, 2, 1, 16, 12, False),
    ("decode_gqa4", 1, 16, 4, 40, 64, 13, False),
    ("decode_gqa6", 1, 12, 2, 201, 256, 14, False),
    ("verify_4rows", 4, 12, 2, 50, 64, 15, False),
    ("prefill_8rows", 8, 4, 2, 0, 16, 16, False),
    ("chunk_19rows", 19, 2, 1, 5, 32, 17, False),
    ("mrope_rows", 3, 4, 2, 7, 16, 18, True),
    ("deep_position", 1, 4, 1, 300, 304, 19, False),   # cache of 300 keys, RoPE at 262000
]


def case_inputs(rows, q_heads, kv_heads, base_pos, max_ctx, seed, multimodal, name=""):
    rng = np.random.default_rng(seed)
    qg, k, v = synth.step_inputs(rng, rows, q_heads, kv_heads)
    kc = np.zeros((kv_heads, max_ctx, 256), np.uint16)
    vc = np.zeros((kv_heads, max_ctx, 256), np.uint16)
    if base_pos:
        kc[:, :base_pos] = synth.cache_bits(rng, kv_heads, base_pos)
        vc[:, :base_pos] = synth.cache_bits(rng, kv_heads, base_pos)
    # stale slots past what this step writes, as tests/test_attn.c:89-97 poisons them
    kc[:, base_pos + rows:] = synth.f32_to_bf16_bits(np.float32([30.0]))[0]
    vc[:, base_pos + rows:] = synth.f32_to_bf16_bits(np.float32([-999.0]))[0]
    pos = synth.positions(262000 if name == "deep_position" else base_pos, rows)
    if multimodal:
        pos[1] = 7 + np.arange(rows)
        pos[2] = 40 + np.arange(rows)
    w = synth.f32_to_bf16_bits(1.0 + 0.25 * rng.standard_normal(256).astype(np.float32))
    return qg, k, v, kc, vc, pos, w


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main():
    from oracle.oracle import Oracle, RefCpu, BF16, F16
    ref_b, ref_h, orc = RefCpu("bf16"), RefCpu("f16"), Oracle()
    axis, inv = ref_b.rope_tables(64, 1e7, (11, 11, 10))
    out = {"rope_axis": axis, "rope_inv_freq": inv}
    for (name, rows, qh, kvh, base, ctx, seed, mm) in CASES:
        qg, k, v, kc, vc, pos, w = case_inputs(rows, qh, kvh, base, ctx, seed, mm, name)
        out[name + "/input_sha256"] = np.frombuffer(bytes.fromhex(digest(qg, k, v, kc, vc, pos, w)), np.uint8)
        kcb, vcb = kc.copy(), vc.copy()
        pre, gate, q_post, k_post = ref_b.attn_layer(qg, k, v, w, w, pos, axis, inv, kcb, vcb, rows, qh, kvh, 256, 64,
                                                     ctx, base, 1e-6, 0.0625, threads=1)
        out[name + "/q_post"] = q_post
        out[name + "/k_post"] = k_post
        out[name + "/kc_rows"] = kcb[:, base:base + rows].copy()
        out[name + "/vc_rows"] = vcb[:, base:base + rows].copy()
        out[name + "/attn_pre_gate"] = pre
        # the same step with the shipped cache type (IEEE half): history converted value for value
        kch = orc.to_cache(orc.from_cache(kc, BF16), F16)
        vch = orc.to_cache(orc.from_cache(vc, BF16), F16)
        pre_h, _, _, _ = ref_h.attn_layer(qg, k, v, w, w, pos, axis, inv, kch, vch, rows, qh, kvh, 256, 64,
                                          ctx, base, 1e-6, 0.0625, threads=1)
        out[name + "/attn_pre_gate_f16"] = pre_h
    path = os.path.join(HERE, "attn_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
