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

`value` is measured with every input already in HBM (CUDA events on the launching stream,
no per-kernel instrumentation; the K steps are one timed region, and the median of the
steps' own intervals is given beside it); the roofline figure of the dominant kernel comes
from a second, instrumented pass.  `e2e` is the same step driven through the
reference-facing ops with HOST buffers, the host->device copies of each layer's q/k/v and
the device->host copy of its output inside the timed region.  Inputs are far larger than
L2 (1.07 GB of K/V per layer, 17 GB per step), so no flush is needed between iterations.

Multi-GPU (one process per GPU, torchrun).  The headline is weak scaling: KV heads are
sharded over min(N, kv_heads) GPUs -- the natural sharding, no collective inside attention
-- and the batch grows with N so that each GPU streams the same bytes; groups beyond
kv_heads GPUs are independent replicas.  Every line also carries, in `extra`:
  strong     config 3 at a FIXED global batch (8, and 1) with heads over min(N, 4) GPUs;
  seq_split  config 5 (262144 keys, batch 1 and 4) with the positions split over min(N, 8)
             GPUs, the ranks' partials exchanged by the library's own peer stores
             (qw_op_attn_exchange), with and without the exchange;
and `parity`: before anything is timed, small cases run through both sharded paths on the
N GPUs and are compared with outputs of the reference's CPU code (tests/golden/
bench_parity.npz); the run fails above 1e-2.
"""
from __future__ import annotations

import argparse
import hashlib
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

from qwasar_b200 import sharding, synth  # noqa: E402

METRIC = "attn decode KV-read GB/s @32K ctx"
UNIT = "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one qw_attn_split_kernel launch, as a
# multiple of the launch's algorithmic K+V bytes: 1.0755 GB read + 4.2 to 4.7 MB written against
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
    head) pairs.  The thread count is the number of cores this process may run on, whatever
    OMP_NUM_THREADS says (torchrun sets it to 1 for its ranks)."""

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
        try:
            self.threads = len(os.sched_getaffinity(0))
        except AttributeError:
            self.threads = os.cpu_count() or 1
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
    """The reference arm: rank 0 alone, in this process, with all the host's cores."""
    if int(os.environ.get("RANK", "0")) != 0:
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
                       "note": "attention only (qw_cpu_attn_decode), built with the reference's -O3 -ffast-math; "
                               "one process on the host's cores at every --gpus"},
            "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": cs.threads, "kind": cs.kind, "sample": sample},
            "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# this library
# ------------------------------------------------------------------------------------------
def rope_tab(be):
    """Device buffer: axis at 0, inv_freq at 128, unit norm weights (bf16) at 512."""
    ax = np.zeros(32, np.uint8); iv = np.zeros(32, np.float32)
    sec = np.asarray(synth.MROPE_SECTION, np.int32)
    be.rope_tables(ax.ctypes.data, iv.ctypes.data, 64, synth.ROPE_THETA, sec.ctypes.data)
    tab = be.buf_alloc_device(1024)
    be.buf_upload(tab, 0, ax); be.buf_upload(tab, 128, iv)
    be.buf_upload(tab, 512, synth.f32_to_bf16_bits(np.ones(256, np.float32)))
    return tab


def fill_random(be, torch, gen, device, karena, varena, layers, kv_heads, ctx, lo, hi):
    """N(0,1) keys and values at positions [lo, hi) of every layer, through the library's own
    append kernel from device data."""
    from qwasar_b200.backend import QwRef
    chunk = 4096
    layer_bytes = kv_heads * ctx * 512
    kf = torch.empty((chunk, kv_heads, 256), dtype=torch.float32, device=device)
    vf = torch.empty_like(kf)
    kfb = be.buf_wrap_device(kf.data_ptr(), kf.numel() * 4); vfb = be.buf_wrap_device(vf.data_ptr(), vf.numel() * 4)
    c = be.cmd_begin(torch.cuda.current_stream().cuda_stream)
    for l in range(layers):
        for t0 in range(lo, hi, chunk):
            n = min(chunk, hi - t0)
            kf.normal_(generator=gen); vf.normal_(generator=gen)
            be.op_kv_write(c, QwRef(karena, l * layer_bytes), QwRef(varena, l * layer_bytes), QwRef(kfb, 0), QwRef(vfb, 0),
                           n, kv_heads, 256, ctx, t0)
    be.cmd_wait(c); be.cmd_free(c)
    be.buf_free(kfb); be.buf_free(vfb)


class DecodeBench:
    """Per-GPU state of the decode / verify workloads: every sequence's K and V arena in one page
    pool, one step's activations, pre-built argument lists for the per-layer batched fused call."""

    def __init__(self, be, torch, wl, n_seq, q_heads, kv_heads, layers, device, host_io, cache="pool"):
        from qwasar_b200.backend import QwRef, BF16
        import ctypes as C
        self.be, self.torch, self.wl = be, torch, wl
        self.n_seq, self.qh, self.kvh, self.layers = n_seq, q_heads, kv_heads, layers
        self.host_io = host_io
        rows, base = wl["rows"], wl["base_pos"]
        self.rows, self.base = rows, base
        self.ctx = ctx = base + rows + 56
        g = torch.Generator(device=device); g.manual_seed(wl["seed"])
        layer_bytes = kv_heads * ctx * 512
        self.pool = None
        if cache == "pool":     # one pool per GPU: all sequences share its pages and its tensor maps
            pages = 2 * n_seq * layers * kv_heads * ((ctx + 63) // 64)
            self.pool = be.kv_pool_alloc(pages * 32768)
            self.karena = [be.kv_arena_alloc_in(self.pool, layers, kv_heads, ctx) for _ in range(n_seq)]
            self.varena = [be.kv_arena_alloc_in(self.pool, layers, kv_heads, ctx) for _ in range(n_seq)]
        elif cache == "arena":  # an arena with a private pool per sequence
            self.karena = [be.kv_arena_alloc(layers, kv_heads, ctx) for _ in range(n_seq)]
            self.varena = [be.kv_arena_alloc(layers, kv_heads, ctx) for _ in range(n_seq)]
        else:                   # the reference's head-major layout in plain device buffers
            self.karena = [be.buf_alloc_device(layers * layer_bytes) for _ in range(n_seq)]
            self.varena = [be.buf_alloc_device(layers * layer_bytes) for _ in range(n_seq)]
        for s in range(n_seq):
            fill_random(be, torch, g, device, self.karena[s], self.varena[s], layers, kv_heads, ctx, 0, base)
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
        self.tab = rope_tab(be)
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
            if self.host_io:            # the layer's output may start its way back to the host (qw_cmd_flush, as the
                self.be.cmd_flush(c)    # reference's graph flushes between layers): it travels under the next layers

    def free(self):
        for b in self.karena + self.varena + self.in_bufs + self.out_bufs + [self.tab]:
            self.be.buf_free(b)
        if self.pool:
            self.be.buf_free(self.pool)


def time_device(be, torch, encode, steps, warmup, barrier):
    """K steps on one stream as ONE timed region (CUDA events on that stream), plus an event after
    every step; returns (ms per step of the region, the steps' own intervals in ms)."""
    stream = torch.cuda.Stream()
    c = be.cmd_begin(stream.cuda_stream)
    for _ in range(warmup):
        encode(c)
    be.cmd_wait(c)
    barrier(); torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record(stream)
    for i in range(steps):
        encode(c)
        marks[i + 1].record(stream)
    be.cmd_wait(c)
    torch.cuda.synchronize(); barrier()
    be.cmd_free(c)
    each = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
    return marks[0].elapsed_time(marks[steps]) / steps, each


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


def kernel_pass(be, torch, encode, steps, warmup, kernel="qw_attn_split"):
    """A separate, instrumented pass: every launch of `kernel` bracketed by CUDA events on its
    stream (which serialises the chain, so this pass gives no step time).  (ms total, launches)."""
    be.prof_kernels(True); be.prof_kernel_read(kernel, True)
    time_device(be, torch, encode, steps, warmup, lambda: None)
    be.prof_kernels(False)
    return be.prof_kernel_read(kernel, True)


def max_over_ranks(torch, dist, world, device, x):
    t = torch.tensor([x], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ---- parity of the sharded paths, before anything is timed ------------------------------------
def _digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest(), np.uint8)


def _rel(got, want):
    num = np.max(np.abs(got.astype(np.float64) - want), axis=-1)
    den = np.maximum(np.max(np.abs(want), axis=-1), 1e-30)
    return float(np.max(num / den))


def parity_block(be, torch, dist, world, rank, device):
    """Small cases through the two sharded paths on all `world` GPUs, against what the reference's
    CPU code returned for the same seeded inputs (tests/golden/bench_parity.npz, made by
    tests/golden/make_bench_parity.py).  Max relative error per output vector, over the gathered
    result; appended K / V rows bit for bit."""
    from qwasar_b200.backend import QwRef, BF16, F32
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_bench_parity as fx
    gold = np.load(os.path.join(ROOT, "tests", "golden", "bench_parity.npz"))
    tab = rope_tab(be)
    res = {}

    def gather(local):          # concatenation over ranks along the head axis, on rank 0's host
        if world == 1:
            return [local]
        local = np.ascontiguousarray(local)
        t = torch.from_numpy(local.view(np.uint8)).to(device)      # as bytes: NCCL carries no 16-bit unsigned type
        outs = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(outs, t)
        return [o.cpu().numpy().view(local.dtype).reshape(local.shape) for o in outs]

    # (1) KV heads sharded: the fused node on each rank's head slice
    for name in ("heads_decode", "heads_verify"):
        case = fx.CASES[name]
        qg, k, v, kc, vc, pos = fx.case_inputs(case)
        assert np.array_equal(_digest(qg, k, v, kc, vc, pos), gold[name + "/input_sha256"]), "parity inputs differ from the fixture's"
        rows, qh, kvh, base = case["rows"], case["q_heads"], case["kv_heads"], case["base_pos"]
        hs, _, _ = sharding.plan(world, kvh, 1)
        _, hshard, _ = sharding.rank_coords(rank, world, kvh, 1)
        (q0, q1), (k0, k1) = sharding.head_slice(hshard, hs, qh, kvh)
        ql, kl, ctx = q1 - q0, k1 - k0, base + rows + 7
        ka, va = be.kv_arena_alloc(1, kl, ctx), be.kv_arena_alloc(1, kl, ctx)
        for h in range(kl):
            be.kv_store(ka, 0, h, 0, kc[k0 + h], kl, ctx); be.kv_store(va, 0, h, 0, vc[k0 + h], kl, ctx)
        bufs = [be.buf_alloc(max(a.nbytes, 16)) for a in (qg[:, q0:q1], k[:, k0:k1], v[:, k0:k1], pos)]
        for b, a in zip(bufs, (qg[:, q0:q1], k[:, k0:k1], v[:, k0:k1], pos)):
            a = np.ascontiguousarray(a)
            be.view(b, a.dtype, a.size)[...] = a.ravel()
        ob = be.buf_alloc(rows * ql * 256 * 4)
        c = be.cmd_begin()
        ok = be.op_attn_layer_fused(c, QwRef(ob, 0), QwRef(bufs[0], 0), QwRef(bufs[1], 0), QwRef(bufs[2], 0), QwRef(tab, 512),
                                    QwRef(tab, 512), QwRef(bufs[3], 0), QwRef(tab, 0), QwRef(tab, 128), QwRef(ka, 0), QwRef(va, 0),
                                    rows, ql, kl, 256, 64, ctx, base, synth.EPS, synth.SCALE, F32)
        if not ok:
            raise RuntimeError("parity: fused node declined: " + str(be.cmd_error(c)))
        be.cmd_wait(c); be.cmd_free(c)
        out_l = np.array(be.view(ob, np.float32, rows * ql * 256)).reshape(rows, ql, 256)
        kr = np.stack([be.kv_read(ka, 0, h, base, rows, kl, ctx) for h in range(kl)])
        vr = np.stack([be.kv_read(va, 0, h, base, rows, kl, ctx) for h in range(kl)])
        outs, krs, vrs = gather(out_l), gather(kr), gather(vr)
        if rank == 0:
            full = np.concatenate(outs[:hs], axis=1)
            res[name + "_max_rel_err"] = _rel(full, gold[name + "/out"])
            res[name + "_kv_rows_bit_exact"] = bool(np.array_equal(np.concatenate(krs[:hs], axis=0), gold[name + "/k_rows"]) and
                                                    np.array_equal(np.concatenate(vrs[:hs], axis=0), gold[name + "/v_rows"]))
        for b in bufs + [ob, ka, va]:
            be.buf_free(b)

    # (2) the sequence split: range-mapped arenas -> pre-op on every rank (append on the owner of the
    # new position) -> qw_op_attn_exchange (split-KV partial, peer stores, merge + gate on every rank)
    name = "seq_decode"
    case = fx.CASES[name]
    qg, k, v, kc, vc, pos = fx.case_inputs(case)
    assert np.array_equal(_digest(qg, k, v, kc, vc, pos), gold[name + "/input_sha256"]), "parity inputs differ from the fixture's"
    rows, qh, kvh, base = case["rows"], case["q_heads"], case["kv_heads"], case["base_pos"]
    ss = min(world, 8)
    out_l = None
    if rank < ss:
        xs, handles = seq_exchange_setup(be, torch, dist, world, rank, device, ss, rows * qh, emulate=world == 1)
        n_keys, ctx = base + rows, base + rows + 7
        ranks_here = range(len(xs))                       # one, or (one GPU) all the emulated ranks
        outs_here = []
        state = []
        for r in ranks_here:
            sr = rank if world > 1 else r
            lo, hi = sharding.seq_range(sr, len(xs) if world == 1 else ss, n_keys)
            ka, va = be.kv_arena_alloc(1, kvh, ctx), be.kv_arena_alloc(1, kvh, ctx)
            h_lo, h_hi = lo, min(hi, base)
            if h_hi > h_lo:
                for h in range(kvh):
                    be.kv_store(ka, 0, h, h_lo, kc[h, h_lo:h_hi], kvh, ctx); be.kv_store(va, 0, h, h_lo, vc[h, h_lo:h_hi], kvh, ctx)
            bufs = [be.buf_alloc(max(a.nbytes, 16)) for a in (qg, k, v, pos)]
            for b, a in zip(bufs, (qg, k, v, pos)):
                be.view(b, a.dtype, a.size)[...] = np.ascontiguousarray(a).ravel()
            qb = be.buf_alloc_device(rows * qh * 256 * 2)
            ob = be.buf_alloc(rows * qh * 256 * 4)
            state.append((lo, hi, ka, va, bufs, qb, ob))
        c = be.cmd_begin()
        phases = (0,) if world > 1 else (1, 2)
        for ph in phases:
            for r, (lo, hi, ka, va, bufs, qb, ob) in zip(ranks_here, state):
                owner = lo <= base < hi
                if ph != 2:
                    ok = be.op_attn_preop(c, QwRef(qb, 0), QwRef(bufs[0], 0), QwRef(bufs[1], 0), QwRef(bufs[2], 0), QwRef(tab, 512),
                                          QwRef(tab, 512), QwRef(bufs[3], 0), QwRef(tab, 0), QwRef(tab, 128), QwRef(ka, 0), QwRef(va, 0),
                                          rows, qh, kvh, 256, 64, ctx, base, synth.EPS, F32, owner)
                    if not ok:
                        raise RuntimeError("parity: pre-op declined: " + str(be.cmd_error(c)))
                ok = be.op_attn_exchange(c, xs[r], ph, QwRef(ob, 0), QwRef(bufs[0], 256 * 4), QwRef(qb, 0), QwRef(ka, 0), QwRef(va, 0),
                                         rows, qh, kvh, 256, ctx, base, lo, hi, synth.SCALE, BF16, F32, F32, 512)
                if not ok:
                    raise RuntimeError("parity: exchange declined: " + str(be.cmd_error(c)))
        be.cmd_wait(c); be.cmd_free(c)
        for (lo, hi, ka, va, bufs, qb, ob) in state:
            outs_here.append(np.array(be.view(ob, np.float32, rows * qh * 256)).reshape(rows, qh, 256))
            for b in bufs + [qb, ob, ka, va]:
                be.buf_free(b)
        for x in xs:
            be.xchg_free(x)
        out_l = outs_here
    if world > 1:
        # every rank of the split holds the whole result: the worst of them counts
        mine = max(_rel(o, gold[name + "/out"]) for o in out_l) if out_l else 0.0
        res_seq = max_over_ranks(torch, dist, world, device, mine)
    else:
        res_seq = max(_rel(o, gold[name + "/out"]) for o in out_l)
    if rank == 0:
        res["seq_max_rel_err"] = res_seq
        res["seq_ranks"] = ss if world > 1 else len(out_l)
        res["seq_path"] = "qw_op_attn_exchange, one call per rank" if world > 1 else "publish then collect, emulated ranks on one GPU"
        res["heads_max_rel_err"] = max(res["heads_decode_max_rel_err"], res["heads_verify_max_rel_err"])
        res["reference"] = "tests/golden/bench_parity.npz (the reference's qwasar_cpu.c)"
        worst = max(res["heads_max_rel_err"], res["seq_max_rel_err"])
        if worst > 1e-2 or not (res["heads_decode_kv_rows_bit_exact"] and res["heads_verify_kv_rows_bit_exact"]):
            raise SystemExit("parity failed: " + json.dumps(res))
    be.buf_free(tab)
    return res


def seq_exchange_setup(be, torch, dist, world, rank, device, ss, max_rh, emulate=False):
    """One exchange object per rank of a sequence group, peers attached: across processes by their
    exported handles (all-gathered as bytes), on one GPU (emulate) four objects attached locally."""
    if emulate:
        n = 4
        xs = [be.xchg_create(n, r, max_rh) for r in range(n)]
        for a in range(n):
            for b in range(n):
                if a != b and not be.xchg_attach_local(xs[a], b, xs[b]):
                    raise RuntimeError(be.last_error())
        return xs, None
    group0 = (rank // ss) * ss
    x = be.xchg_create(ss, rank - group0, max_rh)
    h = be.xchg_export(x)
    t = torch.frombuffer(bytearray(h), dtype=torch.uint8).to(device)
    allh = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(allh, t)
    for r in range(ss):
        if group0 + r != rank:
            be.xchg_attach(x, r, bytes(allh[group0 + r].cpu().numpy().tobytes()))
    return [x], None


# ---- side measurements ---------------------------------------------------------------------------
def prefill_extra(be, torch, peaks, device):
    """Config 2 (4096-token causal prefill, 16 Q / 4 KV heads): TFLOP/s of the whole fused node with
    device-resident bf16 inputs, of the tcgen05 kernel alone (instrumented pass), and end to end
    with host buffers.  Two input sets alternate so that L2 (126 MB) cannot hold a repeat's inputs."""
    from qwasar_b200.backend import QwRef, BF16
    wl = synth.WORKLOADS["c2_9b_prefill_4k"]
    rows, qh, kvh = wl["rows"], wl["q_heads"], wl["kv_heads"]
    ctx = rows + 64
    g = torch.Generator(device=device); g.manual_seed(wl["seed"])
    wrap = lambda t: be.buf_wrap_device(t.data_ptr(), t.numel() * t.element_size())
    pos = torch.arange(rows, device=device, dtype=torch.int32).repeat(3, 1).contiguous()
    sets, keep = [], []
    for _ in range(2):
        qg = torch.randn((rows, qh, 512), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        k = torch.randn((rows, kvh, 256), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        v = torch.randn((rows, kvh, 256), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        out = torch.empty((rows, qh, 256), device=device, dtype=torch.bfloat16)
        keep.append((qg, k, v, out))
        sets.append([wrap(t) for t in (qg, k, v, out, pos)] + [be.kv_arena_alloc(1, kvh, ctx), be.kv_arena_alloc(1, kvh, ctx)])
    tab = rope_tab(be)
    turn = [0]

    def encode(c, bufs=None):
        b = bufs or sets[turn[0] & 1]
        turn[0] += 1
        ok = be.op_attn_layer_fused(c, QwRef(b[3], 0), QwRef(b[0], 0), QwRef(b[1], 0), QwRef(b[2], 0),
                                    QwRef(tab, 512), QwRef(tab, 512), QwRef(b[4], 0), QwRef(tab, 0), QwRef(tab, 128),
                                    QwRef(b[5], 0), QwRef(b[6], 0), rows, qh, kvh, 256, 64, ctx, 0, synth.EPS, synth.SCALE, BF16)
        if not ok:
            raise RuntimeError("prefill declined")
    ms, each = time_device(be, torch, encode, 10, 4, lambda: None)
    k_ms, k_n = kernel_pass(be, torch, encode, 6, 2, "qw_attn_prefill")
    fl = synth.prefill_flops(rows, 0, qh)
    tf = fl / (ms * 1e-3) / 1e12
    res = {"workload": "c2_9b_prefill_4k", "ms": round(ms, 4), "ms_median": round(statistics.median(each), 4), "tflops": round(tf, 2),
           "frac_of_bf16_peak": round(tf / peaks["tf"], 4), "peak_tflops": peaks["tf"], "peak": peaks["which"],
           "l2": "two input sets alternate (2 x 117 MB)"}
    if k_n:
        k_tf = fl / (k_ms / k_n * 1e-3) / 1e12
        res["roofline"] = {"bound": "tensor", "kernel": "qw_attn_prefill_kernel", "achieved": round(k_tf, 1), "peak": peaks["tf"],
                           "unit": "TFLOP/s", "frac": round(k_tf / peaks["tf"], 4), "us_per_launch": round(k_ms / k_n * 1e3, 2),
                           "launches_timed": int(k_n), "flop_per_launch": fl}
    # end to end: inputs in pinned host memory, output read back, inside the timed region
    hb = [be.buf_alloc(n) for n in (rows * qh * 512 * 2, rows * kvh * 256 * 2, rows * kvh * 256 * 2, rows * qh * 256 * 2, 3 * rows * 4)]
    for b, t in zip(hb[:3], keep[0][:3]):
        be.view(b, np.uint16)[:t.numel()] = t.view(torch.int16).cpu().numpy().view(np.uint16).ravel()
    be.view(hb[4], np.int32)[:3 * rows] = pos.cpu().numpy().ravel()
    hset = hb + [sets[0][5], sets[0][6]]
    ms_e = time_e2e(be, torch, lambda c: encode(c, hset), 5, 2, lambda: None)
    res["e2e"] = {"ms": round(ms_e, 3), "tflops": round(fl / (ms_e * 1e-3) / 1e12, 2),
                  "h2d_bytes": rows * (qh * 512 + 2 * kvh * 256) * 2 + 3 * rows * 4, "d2h_bytes": rows * qh * 256 * 2}
    for b in [x for s in sets for x in s] + [tab] + hb:
        be.buf_free(b)
    return res


def next_rows_extra(be, torch, peaks, device):
    """Side measurements of the ops either side of the node: the 4-bit affine product at a
    one-token q_proj shape (weight bytes per second, eight weight sets in rotation so that L2
    cannot serve the repeats), and one QSA step at 262 144 cached positions (block scores from
    stored keys, selection of 512 blocks of 4, masked attention of 16 query / 2 KV heads over the
    2 052 listed positions)."""
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
    ms = time_device(be, torch, q4, 5, 3, lambda: None)[0] / sets
    per = w_bytes + 2 * s_bytes
    out["qmat_q4_decode"] = {"k": k, "n": n, "group": group, "us": round(ms * 1e3, 2), "weight_gbs": round(per / 1e9 / (ms * 1e-3), 1),
                             "frac_of_hbm": round(per / 1e9 / (ms * 1e-3) / peaks["hbm"], 4), "peak": peaks["which"]}
    # ---- the same product for the four rows of a speculative verify: one pass over the weights
    x4 = torch.randn((4, k), generator=g, device=device, dtype=torch.float32)
    y4 = torch.empty((4, n), device=device, dtype=torch.float32)
    bx4, by4 = wrap(x4), wrap(y4)

    def q4v(c):
        for i in range(sets):
            be.op_qmat_q4(c, QwRef(by4, 0), QwRef(bx4, 0), QwRef(bw, i * w_bytes), QwRef(bs, i * s_bytes), QwRef(bb, i * s_bytes), k, n, 4, group)
    ms4 = time_device(be, torch, q4v, 5, 3, lambda: None)[0] / sets
    out["qmat_q4_verify"] = {"k": k, "n": n, "rows": 4, "group": group, "us": round(ms4 * 1e3, 2), "weight_gbs": round(per / 1e9 / (ms4 * 1e-3), 1),
                             "frac_of_hbm": round(per / 1e9 / (ms4 * 1e-3) / peaks["hbm"], 4), "peak": peaks["which"]}
    for b in (bw, bs, bb, bx, by, bx4, by4):
        be.buf_free(b)
    del x4, y4
    # ---- q4 product, many tokens (a prefill-side q_proj): the tcgen05 GEMM with the weights dequantised on their way
    rows_p = 4096
    xp = torch.randn((rows_p, k), generator=g, device=device, dtype=torch.float32)
    yp = torch.empty((rows_p, n), device=device, dtype=torch.float32)
    bxp, byp, bw0, bs0, bb0 = wrap(xp), wrap(yp), wrap(w[0]), wrap(sc[0]), wrap(bi[0])
    def q4p(c):
        be.op_qmm_q4(c, QwRef(byp, 0), QwRef(bxp, 0), QwRef(bw0, 0), QwRef(bs0, 0), QwRef(bb0, 0), k, n, rows_p, group)
    ms = time_device(be, torch, q4p, 5, 3, lambda: None)[0]
    tf = 2.0 * rows_p * k * n / (ms * 1e-3) / 1e12
    out["qmm_q4_prefill"] = {"k": k, "n": n, "rows": rows_p, "group": group, "ms": round(ms, 4), "tflops": round(tf, 1),
                             "frac_of_bf16_peak": round(tf / peaks["tf"], 4), "peak": peaks["which"],
                             "operands": "fp16 (x converted, weights dequantised in shared memory), fp32 accumulate"}
    for b in (bxp, byp, bw0, bs0, bb0):
        be.buf_free(b)
    del w, sc, bi, xp, yp
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
    # Each figure is per launch over `reps` back-to-back launches per timed step (like the eight weight sets of the
    # product above): the event the timer records after a step keeps the next launch from starting under the
    # last one, which is how the layers of a decode step follow one another.
    step, reps = {}, 8
    for name, fn in stages.items():
        def repeated(c, fn=fn):
            for _ in range(reps):
                fn(c)
        step[name] = round(time_device(be, torch, repeated, 10, 3, lambda: None)[0] * 1e3 / reps, 2)
    def chain(c):                      # the three stages back to back, as a decode step encodes them
        for _ in range(reps):
            for fn in stages.values():
                fn(c)
    step["chain_us"] = round(time_device(be, torch, chain, 10, 3, lambda: None)[0] * 1e3 / reps, 2)
    step["launches_per_timed_step"] = reps
    step["listed_kv_bytes"] = int(lst[0, 0].item()) * kvh * 1024
    out["qsa_step_262k"] = step
    for b in bufs:
        be.buf_free(b)
    return out


def small_decode_extra(be, torch, peaks, device, name, layers):
    """Configs 1 and 4 at batch 1: step time per layer and, from an instrumented pass, the split-KV
    kernel alone.  `layers` distinct caches are walked in turn so that L2 cannot serve the repeats."""
    wl = synth.WORKLOADS[name]
    b = DecodeBench(be, torch, wl, 1, wl["q_heads"], wl["kv_heads"], layers, device, host_io=False)
    ms, each = time_device(be, torch, b.encode_step, 30, 5, lambda: None)
    k_ms, k_n = kernel_pass(be, torch, b.encode_step, 6, 2)
    per_layer = b.kv_bytes_step / layers
    res = {"us_per_layer": round(ms * 1e3 / layers, 2), "us_per_layer_median": round(statistics.median(each) * 1e3 / layers, 2),
           "gbs": round(b.kv_bytes_step / 1e9 / (ms * 1e-3), 1), "frac_of_hbm": round(b.kv_bytes_step / 1e9 / (ms * 1e-3) / peaks["hbm"], 4),
           "kv_bytes_per_layer": int(per_layer), "layers_walked": layers}
    if k_n:
        res["kernel_us"] = round(k_ms / k_n * 1e3, 2)
        res["kernel_frac_of_hbm"] = round(per_layer / 1e9 / (k_ms / k_n * 1e-3) / peaks["hbm"], 4)
    b.free()
    if name == "c1_9b_decode_4k":
        res["reference_op_order"] = unfused_layer_extra(be, torch, wl, device, layers)
    return res


def unfused_layer_extra(be, torch, wl, device, layers):
    """The same layer as the graph encodes it op by op (qwasar_graph.c:630-659: split, two norms, two
    rotations, cache write, attention, gate -- eight calls through the C ABI, fp32 activations, a
    caller-owned bf16 cache per layer) beside the one fused call the figure above times."""
    from qwasar_b200.backend import QwRef
    rows, qh, kvh, base = wl["rows"], wl["q_heads"], wl["kv_heads"], wl["base_pos"]
    ctx = base + rows + 56
    g = torch.Generator(device=device); g.manual_seed(wl["seed"] + 100)
    wrap = lambda t: be.buf_wrap_device(t.data_ptr(), t.numel() * t.element_size())
    qg = torch.randn((rows, qh, 512), generator=g, device=device, dtype=torch.float32)
    k = torch.randn((rows, kvh, 256), generator=g, device=device, dtype=torch.float32)
    v = torch.randn((rows, kvh, 256), generator=g, device=device, dtype=torch.float32)
    kn = torch.empty_like(k)
    q = torch.empty((rows, qh, 256), device=device, dtype=torch.float32); gate = torch.empty_like(q); out = torch.empty_like(q)
    pos = torch.arange(base, base + rows, device=device, dtype=torch.int32).repeat(3, 1).contiguous()
    kc = torch.randn((layers, kvh, ctx, 256), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    vc = torch.randn((layers, kvh, ctx, 256), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    keep = (qg, k, v, kn, q, gate, out, pos, kc, vc)
    bqg, bk, bv, bkn, bq, bg, bo, bp, bkc, bvc = [wrap(t) for t in keep]
    tab = rope_tab(be)
    layer_bytes = kvh * ctx * 512

    def encode(c):
        for l in range(layers):
            be.op_split_heads2(c, QwRef(bq, 0), QwRef(bg, 0), QwRef(bqg, 0), rows, qh, 256)
            be.op_rms_norm(c, QwRef(bq, 0), QwRef(bq, 0), QwRef(tab, 512), 256, rows * qh, synth.EPS, 1.0)
            be.op_rms_norm(c, QwRef(bkn, 0), QwRef(bk, 0), QwRef(tab, 512), 256, rows * kvh, synth.EPS, 1.0)
            be.op_rope_partial(c, QwRef(bq, 0), QwRef(bp, 0), QwRef(tab, 0), QwRef(tab, 128), rows, qh, 256, 64)
            be.op_rope_partial(c, QwRef(bkn, 0), QwRef(bp, 0), QwRef(tab, 0), QwRef(tab, 128), rows, kvh, 256, 64)
            be.op_kv_write(c, QwRef(bkc, l * layer_bytes), QwRef(bvc, l * layer_bytes), QwRef(bkn, 0), QwRef(bv, 0), rows, kvh, 256, ctx, base)
            be.op_attn(c, QwRef(bo, 0), QwRef(bq, 0), QwRef(bkc, l * layer_bytes), QwRef(bvc, l * layer_bytes), rows, qh, kvh, 256, ctx,
                       base, synth.SCALE)
            be.op_mul_sigmoid(c, QwRef(bo, 0), QwRef(bg, 0), rows * qh * 256)
    n0 = be.launch_count()
    ms, each = time_device(be, torch, encode, 30, 5, lambda: None)
    launches = (be.launch_count() - n0) // (35 * layers)
    for b in (bqg, bk, bv, bkn, bq, bg, bo, bp, bkc, bvc, tab):
        be.buf_free(b)
    del keep
    return {"us_per_layer": round(ms * 1e3 / layers, 2), "us_per_layer_median": round(statistics.median(each) * 1e3 / layers, 2),
            "calls_per_layer": 8, "kernels_per_layer": int(launches), "activations": "fp32", "cache": "caller-owned bf16, one per layer"}


def strong_extra(be, torch, dist, world, rank, device, wl, layers, barrier, peaks, headline):
    """Config 3 as BASELINE.json words it: a FIXED problem (global batch 8, and batch 1) with KV heads
    sharded over min(N, kv_heads) GPUs; beyond that the eight sequences are dealt over the replica
    groups (batch 1 leaves those GPUs idle).  No collective in the timed region."""
    hs, _, replicas = sharding.plan(world, wl["kv_heads"], 1)
    rep, _, _ = sharding.rank_coords(rank, world, wl["kv_heads"], 1)
    qh_l, kvh_l = wl["q_heads"] // hs, wl["kv_heads"] // hs
    out = {"kv_head_shards": hs, "replica_groups": replicas}
    for gb in (8, 1):
        mine = len([s for s in range(gb) if s % replicas == rep])
        key = f"batch{gb}"
        if world == 1 and gb == 8 and headline:
            out[key] = headline
            continue
        b = DecodeBench(be, torch, wl, mine, qh_l, kvh_l, layers, device, host_io=False) if mine else None
        steps = 20 if gb == 8 else 40
        ms, _ = time_device(be, torch, b.encode_step if b else (lambda c: None), steps, 5, barrier)
        ms = max_over_ranks(torch, dist, world, device, ms if b else 0.0)
        total = layers * gb * synth.decode_kv_bytes(wl["base_pos"] + wl["rows"], wl["kv_heads"])
        used = hs * min(replicas, gb)
        out[key] = {"ms_per_step": round(ms, 4), "us_per_layer": round(ms * 1e3 / layers, 2), "gbs": round(total / 1e9 / (ms * 1e-3), 1),
                    "gpus_used": used, "per_gpu_frac_of_hbm": round(total / used / 1e9 / (ms * 1e-3) / peaks["hbm"], 4),
                    "sequences_per_gpu": mine if gb == 8 else 1, "kv_heads_per_gpu": kvh_l}
        if b:
            b.free()
    return out


def seq_split_extra(be, torch, dist, world, rank, device, barrier, peaks, layers):
    """Config 5 (262 144 cached keys, 16 Q / 2 KV heads) with the positions split over min(N, 8) GPUs.
    A step is, per layer: the pre-op on every rank (query norm + RoPE; the owner of position 262144
    also appends K, V), then qw_op_attn_exchange_batch -- split-KV over the rank's own range, the
    (acc, max, sum) records stored straight into every rank's gather buffer, merge + gate on every
    rank.  `kernels_only` is the same without the exchange (each rank merges only its own partial)."""
    from qwasar_b200.backend import QwRef, BF16
    wl = synth.WORKLOADS["c5_flash_decode_262k"]
    qh, kvh, rows, base = wl["q_heads"], wl["kv_heads"], wl["rows"], wl["base_pos"]
    ss = min(world, 8)
    group0 = (rank // ss) * ss
    srank = rank - group0
    n_keys, ctx = base + rows, base + rows + 56
    lo, hi = sharding.seq_range(srank, ss, n_keys)
    owner = lo <= base < hi
    layer_bytes = kvh * ctx * 512
    out = {"seq_shards": ss, "layers_walked": layers, "keys_per_gpu": hi - lo}
    tab = rope_tab(be)
    for nb in (1, 4):
        gen = torch.Generator(device=device); gen.manual_seed(wl["seed"] + 17 * rank + nb)
        pages = 2 * nb * layers * kvh * ((hi - lo + 63) // 64 + 2)
        pool = be.kv_pool_alloc(pages * 32768)
        kas = [be.kv_arena_alloc_in(pool, layers, kvh, ctx) for _ in range(nb)]
        vas = [be.kv_arena_alloc_in(pool, layers, kvh, ctx) for _ in range(nb)]
        for s in range(nb):
            fill_random(be, torch, gen, device, kas[s], vas[s], layers, kvh, ctx, lo, min(hi, base))
        n_rh = rows * qh
        qg = torch.randn((nb, rows, qh, 512), generator=gen, device=device).to(torch.bfloat16)
        kk = torch.randn((nb, rows, kvh, 256), generator=gen, device=device).to(torch.bfloat16)
        vv = torch.randn((nb, rows, kvh, 256), generator=gen, device=device).to(torch.bfloat16)
        pos = torch.full((3, rows), base, device=device, dtype=torch.int32)
        qn = torch.empty((nb, rows, qh, 256), device=device, dtype=torch.bfloat16)
        o = torch.empty((nb, rows, qh, 256), device=device, dtype=torch.bfloat16)
        pa = torch.empty((nb, n_rh, 258), device=device, dtype=torch.float32)
        W = lambda t: be.buf_wrap_device(t.data_ptr(), t.numel() * t.element_size())
        bqg, bk, bv, bpos, bqn, bo, bpa = [W(t) for t in (qg, kk, vv, pos, qn, o, pa)]
        xs, _ = seq_exchange_setup(be, torch, dist, world, rank, device, ss, nb * n_rh) if world > 1 else ([be.xchg_create(1, 0, nb * n_rh)], None)
        x = xs[0]
        w = QwRef(tab, 512)

        # argument lists are built once: at tens of microseconds per layer the host must not be the clock
        import ctypes as C
        keep, pre_calls, ex_calls, part_calls, merge_calls = [], [], [], [], []

        def refs(fn):
            a = (QwRef * nb)(*[fn(s) for s in range(nb)]); keep.append(a); return C.addressof(a)

        def ints(v):
            a = (C.c_int32 * nb)(*([v] * nb)); keep.append(a); return C.addressof(a)
        for l in range(layers):
            pre_calls.append([(QwRef(bqn, s * n_rh * 512), QwRef(bqg, s * n_rh * 1024), QwRef(bk, s * rows * kvh * 512),
                               QwRef(bv, s * rows * kvh * 512), w, w, QwRef(bpos, 0), QwRef(tab, 0), QwRef(tab, 128),
                               QwRef(kas[s], l * layer_bytes), QwRef(vas[s], l * layer_bytes), rows, qh, kvh, 256, 64, ctx,
                               base, synth.EPS, BF16, owner) for s in range(nb)])
            ex_calls.append((x, 0, nb, refs(lambda s: QwRef(bo, s * n_rh * 512)), refs(lambda s: QwRef(bqg, s * n_rh * 1024 + 512)),
                             refs(lambda s: QwRef(bqn, s * n_rh * 512)), refs(lambda s: QwRef(kas[s], l * layer_bytes)),
                             refs(lambda s: QwRef(vas[s], l * layer_bytes)), ints(base), ints(lo), ints(hi),
                             rows, qh, kvh, 256, ctx, synth.SCALE, BF16, BF16, BF16, 512))
            part_calls.append([(QwRef(bpa, s * n_rh * 258 * 4), QwRef(bpa, (s * n_rh * 258 + n_rh * 256) * 4), QwRef(bqn, s * n_rh * 512),
                                QwRef(kas[s], l * layer_bytes), QwRef(vas[s], l * layer_bytes), rows, qh, kvh, 256, ctx, base, lo, hi,
                                synth.SCALE, BF16) for s in range(nb)])
            merge_calls.append([(QwRef(bo, s * n_rh * 512), QwRef(bpa, s * n_rh * 258 * 4), QwRef(bpa, (s * n_rh * 258 + n_rh * 256) * 4),
                                 QwRef(bqg, s * n_rh * 1024 + 512), rows, qh, 256, 1, 512, BF16, BF16, 0) for s in range(nb)])
        lib = be.lib

        def step(c, exchange):
            for l in range(layers):
                for a in pre_calls[l]:
                    if not lib.qw_op_attn_preop(c, *a):
                        raise RuntimeError("pre-op declined: " + str(be.cmd_error(c)))
                if exchange:
                    if not lib.qw_op_attn_exchange_batch(c, *ex_calls[l]):
                        raise RuntimeError("exchange declined: " + str(be.cmd_error(c)))
                else:
                    for a, m in zip(part_calls[l], merge_calls[l]):
                        if not lib.qw_op_attn_partial(c, *a):
                            raise RuntimeError("partial declined: " + str(be.cmd_error(c)))
                        lib.qw_op_attn_merge(c, *m)

        res = {}
        for name, ex in (("exchange", True), ("kernels_only", False)):
            ms, each = time_device(be, torch, lambda c: step(c, ex), 30, 5, barrier)
            res[name] = max_over_ranks(torch, dist, world, device, ms)
            res[name + "_median"] = max_over_ranks(torch, dist, world, device, statistics.median(each))
        total = layers * nb * synth.decode_kv_bytes(n_keys, kvh)
        out[f"batch{nb}"] = {
            "us_per_layer": round(res["exchange"] * 1e3 / layers, 2), "us_per_layer_median": round(res["exchange_median"] * 1e3 / layers, 2),
            "kernels_only_us_per_layer": round(res["kernels_only"] * 1e3 / layers, 2),
            "gbs": round(total / 1e9 / (res["exchange"] * 1e-3), 1),
            "per_gpu_frac_of_hbm": round(total / ss / 1e9 / (res["exchange"] * 1e-3) / peaks["hbm"], 4),
            "kernels_only_per_gpu_frac_of_hbm": round(total / ss / 1e9 / (res["kernels_only"] * 1e-3) / peaks["hbm"], 4)}
        if nb > 1:      # (why this figure can exceed the step with the exchange)
            out[f"batch{nb}"]["kernels_only_path"] = "qw_op_attn_partial + qw_op_attn_merge once per sequence: the batched form exists only with the exchange"
        for b in (bqg, bk, bv, bpos, bqn, bo, bpa):
            be.buf_free(b)
        be.xchg_free(x)
        for b in kas + vas + [pool]:
            be.buf_free(b)
        del qg, kk, vv, qn, o, pa
    be.buf_free(tab)
    out["exchange"] = "peer stores of the (acc, max, sum) records + flags (qw_op_attn_exchange_batch); no library collective"
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
    if args.only:                      # one side measurement alone: a short run for a profiler to sit on
        fn = {"prefill": lambda: prefill_extra(be, torch, peaks, device),
              "next": lambda: next_rows_extra(be, torch, peaks, device),
              "c1": lambda: small_decode_extra(be, torch, peaks, device, "c1_9b_decode_4k", 16),
              "c4": lambda: small_decode_extra(be, torch, peaks, device, "c4_27b_verify_32k", 8)}[args.only]
        if rank == 0:
            print(json.dumps({"only": args.only, "result": fn()}), flush=True)
        return
    wl = synth.WORKLOADS[args.workload]
    warm = max(3, args.warmup)

    parity = None if args.no_parity else parity_block(be, torch, dist, world, rank, device)

    # weak scaling: heads sharded over hs GPUs, batch grown by hs so per-GPU bytes stay fixed
    hs, _, replicas = sharding.plan(world, wl["kv_heads"], 1)
    batch = args.batch or max(wl["batch"])
    n_seq_local = batch * hs
    qh_l, kvh_l = wl["q_heads"] // hs, wl["kv_heads"] // hs
    layers = args.layers or wl["layers"]

    bench = DecodeBench(be, torch, wl, n_seq_local, qh_l, kvh_l, layers, device, host_io=False, cache=args.cache)
    sampler = ClockSampler(local)
    launches0 = be.launch_count()
    if rank == 0:
        sampler.start()
    ms, each = time_device(be, torch, bench.encode_step, args.steps, warm, barrier)
    if rank == 0 and not sampler.rows and sampler.proc:
        # a short run (few steps) can end before the first 200 ms sample: the same step is repeated, untimed, under
        # the sampler until one has landed, so that the line always carries clocks seen under this load
        t_end = time.time() + 3.0
        while not sampler.rows and time.time() < t_end:
            time_device(be, torch, bench.encode_step, 10, 0, lambda: None)
        sampler.repeated = True
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = ("warm-up and timed steps plus untimed repeats of the step (the run was shorter than one sampling period)"
                            if getattr(sampler, "repeated", False) else "warm-up and timed steps")
    launches = be.launch_count() - launches0
    launches -= (warm * launches) // (warm + args.steps)
    ms_max = max_over_ranks(torch, dist, world, device, ms)
    ms_med = max_over_ranks(torch, dist, world, device, statistics.median(each))
    total_bytes = bench.kv_bytes_step * world
    value = total_bytes / 1e9 / (ms_max * 1e-3)
    # roofline of the dominant kernel on this rank: a second pass with per-launch events
    k_ms, k_n = kernel_pass(be, torch, bench.encode_step, 5, 2)
    k_bytes = bench.kv_bytes_step * 7 / max(1, k_n)
    achieved = k_bytes / 1e9 / (k_ms / max(1, k_n) * 1e-3) if k_n else 0.0
    bench.free()

    # end to end with host buffers
    bench2 = DecodeBench(be, torch, wl, n_seq_local, qh_l, kvh_l, layers, device, host_io=True, cache=args.cache)
    e2e_steps = max(3, min(args.steps, 30))
    ms_e = max_over_ranks(torch, dist, world, device, time_e2e(be, torch, bench2.encode_step, e2e_steps, 2, barrier))
    e2e_value = total_bytes / 1e9 / (ms_e * 1e-3)
    h2d, d2h = bench2.h2d, bench2.d2h
    bench2.free()

    extra = {}
    cpu = None
    if not args.no_extras:
        headline = {"ms_per_step": round(ms_max, 4), "us_per_layer": round(ms_max * 1e3 / layers, 2), "gbs": round(value, 1), "gpus_used": 1,
                    "per_gpu_frac_of_hbm": round(value / peaks["hbm"], 4), "sequences_per_gpu": batch, "kv_heads_per_gpu": kvh_l} if world == 1 else None
        try:
            extra["strong"] = strong_extra(be, torch, dist, world, rank, device, wl, layers, barrier, peaks, headline)
        except Exception as e:   # a side measurement must not lose the headline line
            extra["strong"] = {"error": str(e)[:200]}
        try:
            extra["seq_split"] = seq_split_extra(be, torch, dist, world, rank, device, barrier, peaks, args.seq_layers)
        except Exception as e:
            extra["seq_split"] = {"error": str(e)[:200]}
    if rank == 0 and world == 1 and not args.no_extras:
        for key, fn in (("prefill", lambda: prefill_extra(be, torch, peaks, device)),
                        ("c1_9b_decode_4k", lambda: small_decode_extra(be, torch, peaks, device, "c1_9b_decode_4k", 16)),
                        ("c4_27b_verify_32k", lambda: small_decode_extra(be, torch, peaks, device, "c4_27b_verify_32k", 8))):
            try:
                extra[key] = fn()
            except Exception as e:
                extra[key] = {"error": str(e)[:200]}
        try:
            extra.update(next_rows_extra(be, torch, peaks, device))
        except Exception as e:
            extra["next_rows"] = {"error": str(e)[:200]}
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
            "warmup": warm, "ms_per_step": round(ms_max, 4), "ms_per_step_median": round(ms_med, 4),
            "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "q_heads": wl["q_heads"], "kv_heads": wl["kv_heads"], "head_dim": 256,
                       "context": wl["base_pos"], "rows": wl["rows"], "layers_per_step": layers,
                       "global_batch": batch * world, "kv_head_shards": hs, "replicas": replicas,
                       "kv_cache": {"pool": "paged bf16 arenas in one page pool per GPU", "arena": "paged bf16 arena per sequence",
                                    "linear": "head-major bf16 buffers"}[args.cache],
                       "l2": "inputs larger than L2 (>=1 GB of K/V per layer)",
                       "timing": "one region of K steps; median of the K steps' own intervals beside it; kernel figures from a separate instrumented pass"},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm"], 4), "frac_of_nominal_8TBs": round(achieved / 8000.0, 4),
                         "kernel": "qw_attn_split_kernel", "launches_timed": k_n,
                         "bytes_per_launch": int(k_bytes), "peak_source": peaks["which"],
                         "traffic": None if TRAFFIC_RATIO is None else int(k_bytes * TRAFFIC_RATIO)},
            "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        if parity:
            line["parity"] = parity
        if cpu:
            line["cpu_baseline"] = cpu
        if extra:
            line["extra"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3_27b_decode_32k", choices=sorted(synth.WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU group (default: the workload's)")
    ap.add_argument("--layers", type=int, default=0, help="attention layers per step (default: the model's)")
    ap.add_argument("--seq-layers", type=int, default=4, help="layer caches the sequence-split side measurement walks")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--only", default="", choices=["", "prefill", "next", "c1", "c4"],
                    help="run ONE of the single-GPU side measurements and print its block alone (for profiling that kernel)")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--cache", default="pool", choices=["pool", "arena", "linear"],
                    help="arenas in one page pool, an arena per sequence, or the reference's plain layout")
    ap.add_argument("--tune", default="", help="diagnostic knobs, e.g. split_kg=4 (see qw_gpu_tune)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)      # in this process at every --gpus: the CPU arm needs no launcher
    if args.gpus > 1 and "RANK" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000), os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    run_ours(args)


if __name__ == "__main__":
    main()
