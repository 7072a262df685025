"""Generates tests/golden/bench_parity.npz: what the reference's own CPU code returns for the small
cases that bench.py runs through its sharded multi-GPU paths before it times anything.

    make -C oracle && python tests/golden/make_bench_parity.py

bench.py regenerates each case's inputs from its seed (`case_inputs`, shared with this script; the
fixture stores a SHA-256 of the input bytes), runs the case on N GPUs -- the fused node with KV
heads sharded over the ranks, and a sequence split over the ranks with the partials exchanged --
and compares the gathered result with the outputs stored here.  The outputs are the composition
of qw_cpu_rms_norm / qw_cpu_rope_partial / qw_cpu_kv_write / qw_cpu_attn_decode in the order of
qwasar_graph.c:630-659 (bf16 cache build of the unmodified qwasar_cpu.c) times the sigmoid of the
gate (metal/act.metal:29-37)."""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from qwasar_b200 import synth  # noqa: E402

# name -> geometry; the head counts are those of the benchmark's workloads, the depths are small
CASES = {
    "heads_decode": dict(rows=1, q_heads=24, kv_heads=4, base_pos=1500, seed=101),    # config 3's heads
    "heads_verify": dict(rows=4, q_heads=24, kv_heads=4, base_pos=700, seed=102),     # config 4's rows
    "seq_decode": dict(rows=1, q_heads=16, kv_heads=2, base_pos=4000, seed=103),      # config 5's heads
}


def case_inputs(case):
    """qg, k, v (bf16-exact float32), cache prefixes as bf16 bits, positions."""
    rng = np.random.default_rng(case["seed"])
    rows, qh, kvh, base = case["rows"], case["q_heads"], case["kv_heads"], case["base_pos"]
    qg, k, v = synth.step_inputs(rng, rows, qh, kvh)
    kc = synth.cache_bits(rng, kvh, base)
    vc = synth.cache_bits(rng, kvh, base)
    return qg, k, v, kc, vc, synth.positions(base, rows)


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest(), np.uint8)


def main():
    from oracle.oracle import Oracle, RefCpu
    ref, orc = RefCpu("bf16"), Oracle()
    axis, inv = ref.rope_tables(64, synth.ROPE_THETA, synth.MROPE_SECTION)
    w = synth.f32_to_bf16_bits(np.ones(256, np.float32))
    out = {}
    for name, case in CASES.items():
        rows, qh, kvh, base = case["rows"], case["q_heads"], case["kv_heads"], case["base_pos"]
        qg, k, v, kc, vc, pos = case_inputs(case)
        ctx = base + rows
        kcb = np.zeros((kvh, ctx, 256), np.uint16); vcb = np.zeros((kvh, ctx, 256), np.uint16)
        kcb[:, :base] = kc; vcb[:, :base] = vc
        pre, gate, _, _ = ref.attn_layer(qg, k, v, w, w, pos, axis, inv, kcb, vcb, rows, qh, kvh, 256, 64, ctx, base,
                                         synth.EPS, synth.SCALE, threads=1)
        out[name + "/input_sha256"] = digest(qg, k, v, kc, vc, pos)
        out[name + "/out"] = orc.mul_sigmoid(pre, gate).astype(np.float32)
        out[name + "/k_rows"] = kcb[:, base:].copy()
        out[name + "/v_rows"] = vcb[:, base:].copy()
    path = os.path.join(HERE, "bench_parity.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
