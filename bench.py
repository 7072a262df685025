#!/usr/bin/env python
"""Benchmark of the gated GQA attention path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library (CUDA, C ABI)
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU code, host cores

Headline workload (--workload c3_27b_decode_32k): one decode step of the Qwen3.8-27B
geometry -- 24 query / 4 KV heads, head_dim 256 -- at 32768 cached tokens, batch 8
independent sequences, across the model's 16 full-attention layers (the reference's own
attention bench also runs "16 layers to a command buffer", tools/bench/attnbench.c).  A
step is: per layer, the fused node (split [q|gate], q/k RMS norm, partial RoPE, K/V append
at position 32768, causal attention over 32769 keys, sigmoid gate) for all sequences.
Metric: unique K+V bytes read per second (tools/bench/attnbench.c:45's formula).

`value` is measured with every input already in HBM (CUDA events on the launching stream);
`e2e` is the same step driven through the reference-facing ops with HOST buffers, the
host->device copies of each layer's q/k/v and the device->host copy of its output inside
the timed region.  Inputs are far larger than L2 (1.07 GB of K/V per layer, 17 GB per
step), so no flush is needed between iterations.

Multi-GPU (one process per GPU, torchrun): weak scaling.  KV heads are sharded over
min(N, kv_heads) GPUs -- the natural sharding, no collective inside attention -- and the
batch grows with N so that each GPU streams the same bytes; groups beyond kv_heads GPUs are
independent replicas.  --workload c5_flash_decode_262k --seq-shards S instead splits one
long sequence by position over S GPUs, with the partial (m, l, acc) all-gathered by NCCL
and merged on every rank (strong scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from qwasar_b200 import synth  # noqa: E402

METRIC = "attn decode KV-read GB/s @32K ctx"
UNIT = "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one qw_attn_split_kernel launch, as a
# multiple of the launch's algorithmic K+V bytes: 1.075368 GB read + 4.56 MB written against
# 1.073775 GB (profiles/qw_attn_split_kernel__c3_27b_decode_32k_batch8.md).
TRAFFIC_RATIO = 1.0057


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=float(p["hbm_gbs"]), tf=float(p["bf16_tflops"]), tf_sus=float(p.get("bf16_tflops_sustained", 0)),
                    which="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sus=1400.0, which="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU, sampled every 200 ms while running."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        mhz, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                mhz.append(float(r[0])); mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ------------------------------------------------------------------------------------------
# the reference arm / cpu_baseline: the reference's own scalar attention on the host cores
# ------------------------------------------------------------------------------------------
class CpuSample:
    """qw_cpu_attn_decode (oracle/_ref built with the reference's flags; else the restatement)
    on n_seq sequences of one layer, all host threads over the independent (sequence, row,
    head) pairs."""

    def __init__(self, wl, n_seq):
        from oracle.oracle import Oracle, RefCpu
        self.qh, self.kvh, self.rows, self.base = wl["q_heads"], wl["kv_heads"], wl["rows"], wl["base_pos"]
        self.ctx = self.base + self.rows
        self.n_seq = n_seq
        rng = np.random.default_rng(wl["seed"])
        base_k = synth.cache_bits(rng, self.kvh, self.ctx)
        base_v = synth.cache_bits(rng, self.kvh, self.ctx)
        # distinct caches per sequence at the cost of one draw: rotations of the same values
        self.kcs = [np.ascontiguousarray(np.roll(base_k, 977 * i, axis=1)) for i in range(n_seq)]
        self.vcs = [np.ascontiguousarray(np.roll(base_v, 1409 * i, axis=1)) for i in range(n_seq)]
        self.qs = [synth.normal_bf16(rng, (self.rows, self.qh, 256)) for _ in range(n_seq)]
        if RefCpu.available("bf16_fast"):
            self.impl, self.kind = RefCpu("bf16_fast"), "reference"
        else:
            self.impl, self.kind = Oracle(fast=True), "port"
        self.threads = self.impl.max_threads
        self.gb = n_seq * synth.decode_kv_bytes(self.base + self.rows, self.kvh) / 1e9

    def _one(self, i, threads):
        self.impl.attn_decode(self.qs[i], self.kcs[i], self.vcs[i], self.rows, self.qh, self.kvh, 256, self.ctx,
                              self.base, synth.SCALE, threads=threads)

    def one_pass(self):
        """Seconds for one pass over the n_seq sequences.  Each call spreads its (row, head)
        pairs over OpenMP threads; with fewer pairs than threads several sequences run at once."""
        pairs = max(1, self.rows * self.qh)
        per_call = max(1, min(self.n_seq, self.threads // pairs))
        t0 = time.perf_counter()
        if per_call == 1:
            for i in range(self.n_seq):
                self._one(i, self.threads)
        else:
            import concurrent.futures as cf
            t_each = max(1, self.threads // per_call)
            with cf.ThreadPoolExecutor(per_call) as ex:
                list(ex.map(lambda i: self._one(i, t_each), range(self.n_seq)))
        return time.perf_counter() - t0


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = synth.WORKLOADS[args.workload]
    n_seq = args.batch or max(wl["batch"])
    cs = CpuSample(wl, n_seq)
    sample = f"attention of 1 of {wl['layers']} layers x {n_seq} sequences per step"
    times, t_all = [], time.perf_counter()
    for i in range(args.warmup + args.steps):
        sec = cs.one_pass()
        if i >= args.warmup:
            times.append(sec)
        if time.perf_counter() - t_all > 150 and times:      # keep the whole arm within a few minutes
            break
    sec = statistics.mean(times)
    value = cs.gb / sec
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": args.gpus,
            "steps": len(times), "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over bf16 cache", "data": "synthetic",
            "config": {"workload": args.workload, "batch": n_seq, "layers_per_step": 1,
                       "note": "attention only (qw_cpu_attn_decode), built with the reference's -O3 -ffast-math"},
            "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": cs.threads, "kind": cs.kind, "sample": sample},
            "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# this library
# ------------------------------------------------------------------------------------------
class DecodeBench:
    """Per-GPU state of the decode / verify workloads: caches in paged arenas, one step's
    activations, pre-built argument lists for the per-layer batched fused call."""

    def __init__(self, be, torch, wl, n_seq, q_heads, kv_heads, layers, device, host_io, cache="arena"):
        from qwasar_b200.backend import QwRef, BF16
        import ctypes as C
        self.be, self.torch, self.wl = be, torch, wl
        self.n_seq, self.qh, self.kvh, self.layers = n_seq, q_heads, kv_heads, layers
        rows, base = wl["rows"], wl["base_pos"]
        self.rows, self.base = rows, base
        self.ctx = ctx = base + rows + 56
        g = torch.Generator(device=device); g.manual_seed(wl["seed"])
        # caches: one K and one V arena per sequence, `layers` layers each, filled through the
        # library's own append kernel from N(0,1) device data
        layer_bytes = kv_heads * ctx * 512
        if cache == "arena":
            self.karena = [be.kv_arena_alloc(layers, kv_heads, ctx) for _ in range(n_seq)]
            self.varena = [be.kv_arena_alloc(layers, kv_heads, ctx) for _ in range(n_seq)]
        else:   # the reference's head-major layout in plain device buffers
            self.karena = [be.buf_alloc_device(layers * layer_bytes) for _ in range(n_seq)]
            self.varena = [be.buf_alloc_device(layers * layer_bytes) for _ in range(n_seq)]
        chunk = 4096
        kf = torch.empty((chunk, kv_heads, 256), dtype=torch.float32, device=device)
        vf = torch.empty_like(kf)
        kfb = be.buf_wrap_device(kf.data_ptr(), kf.numel() * 4); vfb = be.buf_wrap_device(vf.data_ptr(), vf.numel() * 4)
        c = be.cmd_begin(torch.cuda.current_stream().cuda_stream)
        for s in range(n_seq):
            for l in range(layers):
                for t0 in range(0, base, chunk):
                    n = min(chunk, base - t0)
                    kf.normal_(generator=g); vf.normal_(generator=g)
                    be.op_kv_write(c, QwRef(self.karena[s], l * layer_bytes), QwRef(self.varena[s], l * layer_bytes),
                                   QwRef(kfb, 0), QwRef(vfb, 0), n, kv_heads, 256, ctx, t0)
        be.cmd_wait(c); be.cmd_free(c)
        be.buf_free(kfb); be.buf_free(vfb)
        del kf, vf
        # activations: per layer one buffer holding every sequence's qg | k | v | pos, and one for out
        self.qg_b = rows * q_heads * 512 * 2; self.k_b = rows * kv_heads * 256 * 2
        self.pos_b = 3 * rows * 4; self.out_b = rows * q_heads * 256 * 2
        self.in_stride = (self.qg_b + 2 * self.k_b + self.pos_b + 255) // 256 * 256
        self.out_stride = (self.out_b + 255) // 256 * 256
        self.h2d = layers * n_seq * (self.qg_b + 2 * self.k_b + self.pos_b)
        self.d2h = layers * n_seq * self.out_b
        rng = np.random.default_rng(wl["seed"] + 1)
        host_in = np.zeros((layers, n_seq * self.in_stride), np.uint8)
        for l in range(layers):
            for s in range(n_seq):
                qg, k, v = synth.step_inputs(rng, rows, q_heads, kv_heads)
                o = s * self.in_stride
                host_in[l, o:o + self.qg_b] = synth.f32_to_bf16_bits(qg).view(np.uint8).ravel(); o += self.qg_b
                host_in[l, o:o + self.k_b] = synth.f32_to_bf16_bits(k).view(np.uint8).ravel(); o += self.k_b
                host_in[l, o:o + self.k_b] = synth.f32_to_bf16_bits(v).view(np.uint8).ravel(); o += self.k_b
                host_in[l, o:o + self.pos_b] = synth.positions(base, rows).view(np.uint8).ravel()
        self.in_bufs, self.out_bufs = [], []
        for l in range(layers):
            if host_io:
                b = be.buf_alloc(host_in.shape[1]); be.view(b, np.uint8)[:host_in.shape[1]] = host_in[l]
                ob = be.buf_alloc(n_seq * self.out_stride)
            else:
                b = be.buf_alloc_device(host_in.shape[1]); be.buf_upload(b, 0, host_in[l])
                ob = be.buf_alloc_device(n_seq * self.out_stride)
            self.in_bufs.append(b); self.out_bufs.append(ob)
        axis, inv = synth.rope_tables()
        ax = np.zeros(32, np.uint8); iv = np.zeros(32, np.float32)
        sec = np.asarray(synth.MROPE_SECTION, np.int32)
        be.rope_tables(ax.ctypes.data, iv.ctypes.data, 64, synth.ROPE_THETA, sec.ctypes.data)
        self.tab = be.buf_alloc_device(1024)
        be.buf_upload(self.tab, 0, ax); be.buf_upload(self.tab, 128, iv)
        be.buf_upload(self.tab, 512, synth.f32_to_bf16_bits(np.ones(256, np.float32)))
        # pre-built argument lists (ctypes arrays are built once, not per step)
        self.calls, self._keep = [], []
        for l in range(layers):
            def arr(fn):
                a = (QwRef * n_seq)(*[fn(s) for s in range(n_seq)]); self._keep.append(a); return C.addressof(a)
            ib, ob = self.in_bufs[l], self.out_bufs[l]
            outs = arr(lambda s: QwRef(ob, s * self.out_stride))
            qgs = arr(lambda s: QwRef(ib, s * self.in_stride))
            ks = arr(lambda s: QwRef(ib, s * self.in_stride + self.qg_b))
            vs = arr(lambda s: QwRef(ib, s * self.in_stride + self.qg_b + self.k_b))
            ps = arr(lambda s: QwRef(ib, s * self.in_stride + self.qg_b + 2 * self.k_b))
            kcs = arr(lambda s: QwRef(self.karena[s], l * layer_bytes))
            vcs = arr(lambda s: QwRef(self.varena[s], l * layer_bytes))
            bp = (C.c_int32 * n_seq)(*([base] * n_seq)); self._keep.append(bp)
            w = QwRef(self.tab, 512)
            self.calls.append((n_seq, outs, qgs, ks, vs, w, w, ps, QwRef(self.tab, 0), QwRef(self.tab, 128), kcs, vcs,
                               C.addressof(bp), rows, q_heads, kv_heads, 256, 64, ctx, synth.EPS, synth.SCALE, BF16))
        self.kv_bytes_step = layers * n_seq * synth.decode_kv_bytes(base + rows, kv_heads)

    def encode_step(self, c):
        f = self.be.lib.qw_op_attn_layer_fused_batch
        for a in self.calls:
            if not f(c, *a):
                raise RuntimeError("fused node declined: " + str(self.be.cmd_error(c)))

    def free(self):
        for b in self.karena + self.varena + self.in_bufs + self.out_bufs + [self.tab]:
            self.be.buf_free(b)


def time_device(be, torch, encode, steps, warmup, barrier):
    """K steps on one stream, CUDA events on that stream; returns ms per step."""
    stream = torch.cuda.Stream()
    c = be.cmd_begin(stream.cuda_stream)
    for _ in range(warmup):
        encode(c)
    be.cmd_wait(c)
    barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        encode(c)
    e1.record(stream)
    be.cmd_wait(c)
    torch.cuda.synchronize(); barrier()
    be.cmd_free(c)
    return e0.elapsed_time(e1) / steps


def time_e2e(be, torch, encode, steps, warmup, barrier):
    """The same step with host buffers: each step is its own command buffer, so every layer's
    inputs are copied host->device and its output device->host inside the timed region."""
    def one():
        c = be.cmd_begin()
        encode(c)
        be.cmd_wait(c); be.cmd_free(c)
    for _ in range(max(1, warmup)):
        one()
    barrier(); torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    barrier()
    return dt * 1e3 / steps


def prefill_extra(be, torch, peaks, device):
    """Config 2 (4096-token causal prefill, 16 Q / 4 KV heads) as a side measurement: TFLOP/s of
    the whole fused node, device-resident bf16 inputs."""
    from qwasar_b200.backend import QwRef, BF16
    wl = synth.WORKLOADS["c2_9b_prefill_4k"]
    rows, qh, kvh = wl["rows"], wl["q_heads"], wl["kv_heads"]
    ctx = rows + 64
    g = torch.Generator(device=device); g.manual_seed(wl["seed"])
    qg = torch.randn((rows, qh, 512), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn((rows, kvh, 256), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn((rows, kvh, 256), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    out = torch.empty((rows, qh, 256), device=device, dtype=torch.bfloat16)
    pos = torch.arange(rows, device=device, dtype=torch.int32).repeat(3, 1).contiguous()
    wrap = lambda t: be.buf_wrap_device(t.data_ptr(), t.numel() * t.element_size())
    bufs = [wrap(t) for t in (qg, k, v, out, pos)]
    ka, va = be.kv_arena_alloc(1, kvh, ctx), be.kv_arena_alloc(1, kvh, ctx)
    tab = be.buf_alloc_device(1024)
    ax = np.zeros(32, np.uint8); iv = np.zeros(32, np.float32); sec = np.asarray(synth.MROPE_SECTION, np.int32)
    be.rope_tables(ax.ctypes.data, iv.ctypes.data, 64, synth.ROPE_THETA, sec.ctypes.data)
    be.buf_upload(tab, 0, ax); be.buf_upload(tab, 128, iv)
    be.buf_upload(tab, 512, synth.f32_to_bf16_bits(np.ones(256, np.float32)))

    def encode(c):
        ok = be.op_attn_layer_fused(c, QwRef(bufs[3], 0), QwRef(bufs[0], 0), QwRef(bufs[1], 0), QwRef(bufs[2], 0),
                                    QwRef(tab, 512), QwRef(tab, 512), QwRef(bufs[4], 0), QwRef(tab, 0), QwRef(tab, 128),
                                    QwRef(ka, 0), QwRef(va, 0), rows, qh, kvh, 256, 64, ctx, 0, synth.EPS, synth.SCALE, BF16)
        if not ok:
            raise RuntimeError("prefill declined")
    ms = time_device(be, torch, encode, 5, 3, lambda: None)
    fl = synth.prefill_flops(rows, 0, qh)
    tf = fl / (ms * 1e-3) / 1e12
    for b in bufs + [ka, va, tab]:
        be.buf_free(b)
    return {"workload": "c2_9b_prefill_4k", "ms": round(ms, 4), "tflops": round(tf, 2),
            "frac_of_bf16_peak": round(tf / peaks["tf"], 4), "peak_tflops": peaks["tf"], "peak": peaks["which"]}


def next_rows_extra(be, torch, peaks, device):
    """Side measurements of the ops either side of the node (first correct versions, not tuned):
    the 4-bit affine product at a one-token q_proj shape (weight bytes per second, eight weight
    sets in rotation so that L2 cannot serve the repeats), and one QSA step at 262 144 cached
    positions (block scores from stored keys, selection of 512 blocks of 4, masked attention of
    16 query / 2 KV heads over the 2 052 listed positions)."""
    from qwasar_b200.backend import QwRef
    out = {}
    wrap = lambda t: be.buf_wrap_device(t.data_ptr(), t.numel() * t.element_size())
    g = torch.Generator(device=device); g.manual_seed(5)
    # ---- q4 product, rows = 1
    k, n, group, sets = 5120, 12288, 64, 8
    w = torch.randint(0, 2 ** 31 - 1, (sets, n, k // 8), generator=g, device=device, dtype=torch.int32)
    sc = (0.02 * torch.randn((sets, n, k // group), generator=g, device=device)).to(torch.bfloat16)
    bi = (0.1 * torch.randn((sets, n, k // group), generator=g, device=device)).to(torch.bfloat16)
    x = torch.randn((1, k), generator=g, device=device, dtype=torch.float32)
    y = torch.empty((1, n), device=device, dtype=torch.float32)
    bw, bs, bb, bx, by = wrap(w), wrap(sc), wrap(bi), wrap(x), wrap(y)
    w_bytes, s_bytes = n * (k // 8) * 4, n * (k // group) * 2

    def q4(c):
        for i in range(sets):
            be.op_qmat_q4(c, QwRef(by, 0), QwRef(bx, 0), QwRef(bw, i * w_bytes), QwRef(bs, i * s_bytes), QwRef(bb, i * s_bytes), k, n, 1, group)
    ms = time_device(be, torch, q4, 5, 3, lambda: None) / sets
    per = w_bytes + 2 * s_bytes
    out["qmat_q4_decode"] = {"k": k, "n": n, "group": group, "us": round(ms * 1e3, 2), "weight_gbs": round(per / 1e9 / (ms * 1e-3), 1),
                             "frac_of_hbm": round(per / 1e9 / (ms * 1e-3) / peaks["hbm"], 4), "peak": peaks["which"]}
    for b in (bw, bs, bb, bx, by):
        be.buf_free(b)
    del w, sc, bi
    # ---- one QSA step at 262 144 positions
    ctx, ratio, topk, nq, d, qh, kvh = 262144 + 64, 4, 512, 4, 128, 16, 2
    base, max_blocks, cap = 262144, (262144 + 64) // 4, 512 * 4 + 4
    pool = torch.randn((max_blocks, d), generator=g, device=device, dtype=torch.float32)
    qn = torch.randn((1, nq, d), generator=g, device=device, dtype=torch.float32)
    scores = torch.zeros((1, max_blocks), device=device, dtype=torch.float32)
    mask = torch.zeros((1, ctx), device=device, dtype=torch.uint8)
    lst = torch.zeros((1, 1 + cap), device=device, dtype=torch.int32)
    q = torch.randn((1, qh, 256), generator=g, device=device, dtype=torch.float32)
    o = torch.empty((1, qh, 256), device=device, dtype=torch.float32)
    kc = torch.randn((kvh, ctx, 256), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    vc = torch.randn((kvh, ctx, 256), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    bufs = [wrap(t) for t in (pool, qn, scores, mask, lst, q, o, kc, vc)]
    bp, bq, bsco, bm, bl, bqq, bo, bk, bv = bufs
    stages = {
        "scores_us": lambda c: be.op_qsa_scores_pooled(c, QwRef(bsco, 0), QwRef(bq, 0), QwRef(bp, 0), 1, nq, d, ratio, base, max_blocks),
        "select_us": lambda c: be.op_qsa_select(c, QwRef(bm, 0), QwRef(bl, 0), QwRef(bsco, 0), 1, ratio, base, topk, ctx, max_blocks),
        "attend_us": lambda c: be.op_attn_masked(c, QwRef(bo, 0), QwRef(bqq, 0), QwRef(bk, 0), QwRef(bv, 0), QwRef(bl, 0), 1, qh, kvh, 256,
                                                 ctx, base, 0.0625, topk, ratio),
    }
    step = {}
    for name, fn in stages.items():
        step[name] = round(time_device(be, torch, fn, 10, 3, lambda: None) * 1e3, 2)
    step["listed_kv_bytes"] = int(lst[0, 0].item()) * kvh * 1024
    out["qsa_step_262k"] = step
    for b in bufs:
        be.buf_free(b)
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    import qwasar_b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    be = qwasar_b200.Backend()
    for kv in filter(None, args.tune.split(",")):
        k, v = kv.split("=")
        if not be.tune(k, int(v)):
            raise SystemExit(f"unknown knob {kv}")
    peaks = measured_peaks()
    wl = synth.WORKLOADS[args.workload]
    if args.seq_shards > 1:
        return run_seq_split(args, be, torch, dist, wl, world, rank, device, peaks, barrier)

    # weak scaling: heads sharded over hs GPUs, batch grown by hs so per-GPU bytes stay fixed
    from qwasar_b200 import sharding
    hs, _, replicas = sharding.plan(world, wl["kv_heads"], 1)
    batch = args.batch or max(wl["batch"])
    n_seq_local = batch * hs
    qh_l, kvh_l = wl["q_heads"] // hs, wl["kv_heads"] // hs
    layers = args.layers or wl["layers"]

    bench = DecodeBench(be, torch, wl, n_seq_local, qh_l, kvh_l, layers, device, host_io=False, cache=args.cache)
    sampler = ClockSampler(local)
    launches0 = be.launch_count()
    be.prof_kernels(True); be.prof_kernel_read("qw_attn_split", True)
    if rank == 0:
        sampler.start()
    ms = time_device(be, torch, bench.encode_step, args.steps, max(3, args.warmup), barrier)
    clocks = sampler.stop() if rank == 0 else None
    be.prof_kernels(False)
    k_ms, k_n = be.prof_kernel_read("qw_attn_split", True)
    launches = be.launch_count() - launches0
    warm_launch = (max(3, args.warmup) * launches) // (max(3, args.warmup) + args.steps)
    launches -= warm_launch
    ms_t = torch.tensor([ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms_max = float(ms_t.item())
    total_bytes = bench.kv_bytes_step * world
    value = total_bytes / 1e9 / (ms_max * 1e-3)
    # roofline of the dominant kernel on this rank (warm-up launches included in the average)
    k_bytes = bench.kv_bytes_step * (max(3, args.warmup) + args.steps) / max(1, k_n)
    achieved = k_bytes / 1e9 / (k_ms / max(1, k_n) * 1e-3) if k_n else 0.0
    bench.free()

    # end to end with host buffers
    bench2 = DecodeBench(be, torch, wl, n_seq_local, qh_l, kvh_l, layers, device, host_io=True)
    e2e_steps = max(3, min(args.steps, 30))
    ms_e = time_e2e(be, torch, bench2.encode_step, e2e_steps, 2, barrier)
    ms_e_t = torch.tensor([ms_e], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms_e_t, op=dist.ReduceOp.MAX)
    e2e_value = total_bytes / 1e9 / (float(ms_e_t.item()) * 1e-3)
    h2d, d2h = bench2.h2d, bench2.d2h
    bench2.free()

    extra = {}
    cpu = None
    if rank == 0 and world == 1 and not args.no_extras:
        try:
            extra["prefill"] = prefill_extra(be, torch, peaks, device)
        except Exception as e:   # the side measurement must not lose the headline line
            extra["prefill"] = {"error": str(e)[:200]}
        try:
            extra.update(next_rows_extra(be, torch, peaks, device))
        except Exception as e:
            extra["next_rows"] = {"error": str(e)[:200]}
        try:
            b1 = DecodeBench(be, torch, wl, 1, wl["q_heads"], wl["kv_heads"], layers, device, host_io=False)
            ms1 = time_device(be, torch, b1.encode_step, max(20, args.steps), 5, barrier)
            extra["batch1"] = {"ms_per_step": round(ms1, 4), "gbs": round(b1.kv_bytes_step / 1e9 / (ms1 * 1e-3), 1),
                               "us_per_layer": round(ms1 * 1e3 / layers, 2)}
            b1.free()
        except Exception as e:
            extra["batch1"] = {"error": str(e)[:200]}
        cs = CpuSample(wl, batch)
        cs.one_pass()
        reps, spent = 0, 0.0
        while spent < 10.0:
            spent += cs.one_pass(); reps += 1
        cpu = {"value": round(cs.gb / (spent / reps), 3), "unit": UNIT, "cores": cs.threads, "kind": cs.kind,
               "sample": f"attention of 1 of {layers} layers x {batch} sequences, {reps} passes of {spent / reps:.2f} s"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": round(ms_max, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "q_heads": wl["q_heads"], "kv_heads": wl["kv_heads"], "head_dim": 256,
                       "context": wl["base_pos"], "rows": wl["rows"], "layers_per_step": layers,
                       "global_batch": batch * world, "kv_head_shards": hs, "replicas": replicas,
                       "kv_cache": "paged bf16 arena" if args.cache == "arena" else "head-major bf16 buffers", "l2": "inputs larger than L2 (>=1 GB of K/V per layer)"},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm"], 4), "frac_of_nominal_8TBs": round(achieved / 8000.0, 4),
                         "kernel": "qw_attn_split_kernel", "launches_timed": k_n,
                         "bytes_per_launch": int(k_bytes), "peak_source": peaks["which"],
                         "traffic": None if TRAFFIC_RATIO is None else int(k_bytes * TRAFFIC_RATIO)},
            "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        if extra:
            line["extra"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_seq_split(args, be, torch, dist, wl, world, rank, device, peaks, barrier):
    """Long-context decode split by position over `seq_shards` GPUs (and by KV heads over the rest):
    every rank holds the keys of its own position range -- its arena maps only those pages --
    computes its partial with qw_op_attn_partial, the ranks of a sequence group all-gather one packed
    record (acc | max, sum) per rank over NCCL, and every rank merges + gates."""
    from qwasar_b200.backend import QwRef, BF16
    from qwasar_b200 import sharding
    ss = args.seq_shards
    hs, _, replicas = sharding.plan(world, wl["kv_heads"], ss)
    rep, hshard, srank = sharding.rank_coords(rank, world, wl["kv_heads"], ss)
    (q0, q1), (k0, k1) = sharding.head_slice(hshard, hs, wl["q_heads"], wl["kv_heads"])
    qh, kvh, rows, base = q1 - q0, k1 - k0, wl["rows"], wl["base_pos"]
    layers = args.layers or wl["layers"]
    ctx = base + rows + 56
    n_keys = base + rows
    lo, hi = sharding.seq_range(srank, ss, n_keys)
    group = None
    if world > 1:
        for g0 in range(0, world, ss):                      # every rank creates every group
            g = dist.new_group(list(range(g0, g0 + ss)))
            if g0 <= rank < g0 + ss:
                group = g
    stream = torch.cuda.Stream()
    gen = torch.Generator(device=device); gen.manual_seed(wl["seed"] + rank)
    layer_bytes = kvh * ctx * 512
    ka, va = be.kv_arena_alloc(layers, kvh, ctx), be.kv_arena_alloc(layers, kvh, ctx)
    chunk = 4096
    kf = torch.empty((chunk, kvh, 256), dtype=torch.float32, device=device); vf = torch.empty_like(kf)
    kfb = be.buf_wrap_device(kf.data_ptr(), kf.numel() * 4); vfb = be.buf_wrap_device(vf.data_ptr(), vf.numel() * 4)
    c = be.cmd_begin(torch.cuda.current_stream().cuda_stream)
    for l in range(layers):
        for t0 in range(lo, hi, chunk):
            n = min(chunk, hi - t0)
            kf.normal_(generator=gen); vf.normal_(generator=gen)
            be.op_kv_write(c, QwRef(ka, l * layer_bytes), QwRef(va, l * layer_bytes), QwRef(kfb, 0), QwRef(vfb, 0),
                           n, kvh, 256, ctx, t0)
    be.cmd_wait(c); be.cmd_free(c)
    be.buf_free(kfb); be.buf_free(vfb)
    committed = be.kv_arena_bytes_committed(ka) + be.kv_arena_bytes_committed(va)
    n_rh = rows * qh
    q = torch.randn((rows, qh, 256), generator=gen, device=device).to(torch.bfloat16)
    gate = torch.randn((rows, qh, 256), generator=gen, device=device).to(torch.bfloat16)
    out = torch.empty((rows, qh, 256), dtype=torch.bfloat16, device=device)
    rec = n_rh * 258                                          # floats per rank: acc block, then stat block
    local = torch.zeros(rec, dtype=torch.float32, device=device)
    gathered = torch.zeros((ss, rec), dtype=torch.float32, device=device)
    W = lambda t: be.buf_wrap_device(t.data_ptr(), t.numel() * t.element_size())
    qb, gb, ob, lb, gbuf = W(q), W(gate), W(out), W(local), W(gathered)

    def step(c, with_collective):
        for l in range(layers):
            ok = be.op_attn_partial(c, QwRef(lb, 0), QwRef(lb, n_rh * 256 * 4), QwRef(qb, 0), QwRef(ka, l * layer_bytes),
                                    QwRef(va, l * layer_bytes), rows, qh, kvh, 256, ctx, base, lo, hi, synth.SCALE, BF16)
            if not ok:
                raise RuntimeError("partial declined: " + str(be.cmd_error(c)))
            if with_collective and ss > 1:
                with torch.cuda.stream(stream):
                    dist.all_gather_into_tensor(gathered, local, group=group)
                be.op_attn_merge(c, QwRef(ob, 0), QwRef(gbuf, 0), QwRef(gbuf, n_rh * 256 * 4), QwRef(gb, 0), rows, qh, 256,
                                 ss, 256, BF16, BF16, rec)
            else:
                be.op_attn_merge(c, QwRef(ob, 0), QwRef(lb, 0), QwRef(lb, n_rh * 256 * 4), QwRef(gb, 0), rows, qh, 256,
                                 1, 256, BF16, BF16, rec)

    res = {}
    for name, coll in (("with_collective", True), ("kernels_only", False)):
        c = be.cmd_begin(stream.cuda_stream)
        for _ in range(max(3, args.warmup)):
            step(c, coll)
        be.cmd_wait(c); barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step(c, coll)
        e1.record(stream)
        be.cmd_wait(c); torch.cuda.synchronize(); barrier()
        be.cmd_free(c)
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name] = float(t.item())
    total_bytes = layers * synth.decode_kv_bytes(n_keys, wl["kv_heads"]) * replicas
    if rank == 0:
        ms = res["with_collective"]
        value = total_bytes / 1e9 / (ms * 1e-3)
        line = {"metric": "attn decode KV-read GB/s, sequence split", "value": round(value, 1), "unit": UNIT,
                "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms, 4),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": args.workload, "seq_shards": ss, "kv_head_shards": hs, "replicas": replicas,
                           "layers_per_step": layers, "batch": 1, "context": base,
                           "collective": "one NCCL all_gather of the packed (acc, max, sum) record per layer",
                           "arena_bytes_committed_rank0": committed},
                "kernels_only_ms_per_step": round(res["kernels_only"], 4),
                "us_per_layer": round(ms * 1e3 / layers, 2), "kernels_only_us_per_layer": round(res["kernels_only"] * 1e3 / layers, 2),
                "per_gpu_frac_of_hbm_kernels_only": round(total_bytes / world / 1e9 / (res["kernels_only"] * 1e-3) / peaks["hbm"], 4),
                "peak_source": peaks["which"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3_27b_decode_32k", choices=sorted(synth.WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU group (default: the workload's)")
    ap.add_argument("--layers", type=int, default=0, help="attention layers per step (default: the model's)")
    ap.add_argument("--seq-shards", type=int, default=1)
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--cache", default="arena", choices=["arena", "linear"], help="paged arena or the reference's plain layout")
    ap.add_argument("--tune", default="", help="diagnostic knobs, e.g. split_kg=4 (see qw_gpu_tune)")
    args = ap.parse_args()
    if args.gpus > 1 and "RANK" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000), os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
