#!/usr/bin/env python
"""Benchmark of the attention hot path (RoPE + KV append + GQA decode attention).

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload cfg5]

One "step" is one decode token through every layer's attention (fused
bias/QK-norm/RoPE/append kernel, split-K decode kernel, split merge) over
synthetic N(0,1) KV caches of the named shape.  The headline `value` is decode
tokens/s with inputs resident in HBM; `e2e` is the same metric through the
host-pointer C-ABI entry (pinned host inputs, H2D and D2H inside the timed
region); `roofline` is the attention kernel's algorithmic HBM bytes over its
device time against the measured copy bandwidth; `cpu_baseline` is the CPU
oracle (a port of the reference's Crystal host path) timed on this host.

`--impl reference` times that CPU port alone (the reference's host language has
no compiler on this image, so its own binary cannot be run).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # BASELINE config 5: Qwen3-30B-A3B-shaped long-context decode attention
    "cfg5": dict(name="cfg5: Qwen3-30B-A3B attention, 48 layers, batch 1, fp32 KV cache ctx 32768, decode",
                 H=32, KV=4, hd=128, theta=1e6, qk_norm=True, layers=48, ctx=32768),
    # BASELINE config 2 (attention part): LLaMA-3.2-1B, 16 layers, ctx 4096
    "cfg2": dict(name="cfg2: LLaMA-3.2-1B attention, 16 layers, batch 1, fp32 KV cache ctx 4096, decode",
                 H=32, KV=8, hd=64, theta=5e5, qk_norm=False, layers=16, ctx=4096),
}
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one attn_decode_fused_kernel launch on the cfg5 shape at
# L = 32770, from an ncu capture of a 4-layer case of the same shape: 139.3 MB for 134.26 MB algorithmic.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 139.3 / 134.26


def decode_bytes(wl, L, kv_heads=None, elem_bytes=4):
    """Algorithmic HBM bytes of one layer-step at visible length L: K and V read
    once, the new row written (cache elements of elem_bytes), q read and out written (fp32)."""
    KV = wl["KV"] if kv_heads is None else kv_heads
    H = wl["H"] * KV // wl["KV"]
    return 2 * KV * L * wl["hd"] * elem_bytes + 2 * KV * wl["hd"] * elem_bytes + 2 * H * wl["hd"] * 4


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed regions run."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.01)

    def start(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t is not None:
            self._t.join()
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def host_threads():
    """Host cores this process may run on.  Asked of the scheduler, not of OpenMP: a launcher
    may have set OMP_NUM_THREADS=1 for its ranks, which would turn the CPU baseline into a
    one-core figure at some rank counts and an all-core figure at others."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_port_rate(wl, threads, layers_sampled, steps, seed=5001):
    """Decode tokens/s of the CPU oracle: `steps` steps of `layers_sampled` layers at
    the workload's context, scaled to the full layer count."""
    from oracle import oracle as O
    rng = np.random.default_rng(seed)
    H, KV, hd = wl["H"], wl["KV"], wl["hd"]
    kw = {}
    if wl["qk_norm"]:
        kw = dict(q_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32),
                  k_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32))
    o = O.OracleAttention(H, KV, hd, wl["theta"], 1e-6, **kw)
    kc = rng.standard_normal((KV, wl["ctx"], hd), dtype=np.float32)
    vc = rng.standard_normal((KV, wl["ctx"], hd), dtype=np.float32)
    o.import_cache(kc, vc)
    q = rng.standard_normal((1, H * hd)).astype(np.float32)
    k = rng.standard_normal((1, KV * hd)).astype(np.float32)
    v = rng.standard_normal((1, KV * hd)).astype(np.float32)
    per_step = []
    for _ in range(steps):
        t0 = time.perf_counter()
        for _ in range(layers_sampled):
            o.attend_cached(q, k, v, threads=threads)
        per_step.append(time.perf_counter() - t0)
    return per_step


def run_reference(args, wl, rank, world):
    if rank != 0:
        return
    threads = host_threads()
    warm = cpu_port_rate(wl, threads, 1, max(1, min(args.warmup, 2)))     # warm-up (page in, thread pool)
    # as many of the layers per step as keep the whole run within about two minutes
    layers_sampled = int(max(1, min(wl["layers"], 120.0 / (max(args.steps, 1) * max(min(warm), 1e-4)))))
    t0 = time.perf_counter()
    per_step = cpu_port_rate(wl, threads, layers_sampled, args.steps)
    wall = time.perf_counter() - t0
    sec_per_token = float(np.sum(per_step)) / args.steps * wl["layers"] / layers_sampled
    value = 1.0 / sec_per_token
    sample = (f"{args.steps} decode steps x {layers_sampled} of {wl['layers']} layers at ctx {wl['ctx']}"
              + ("" if layers_sampled == wl["layers"] else ", scaled to all layers")
              + "; OpenMP over (query head, row block) work items")
    line = {
        "impl": "reference", "metric": "decode_attn_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec_per_token * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"], "timed": "CPU port of the reference's Crystal attention path "
                   "(no Crystal compiler on this image)", "wall_s": wall},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


PREFILL_WL = dict(name="cfg3: Qwen3-8B attention, causal prefill of 8192 tokens, fp32 in / TF32 tensor-core math",
                  H=32, KV=8, hd=128, theta=1e6, S=8192, layers_total=36, layers_timed=2)


def prefill_block(S, ctx, dev, stream_obj):
    """Prefill attention TFLOP/s on the cfg3 shape (norm/RoPE/append kernel + tcgen05
    causal attention kernel per layer), timed with CUDA events on the launching stream.
    Flops are the causal ones: 2*hd*H*S*(S+1) per layer."""
    import torch
    w = PREFILL_WL
    H, KV, hd, T = w["H"], w["KV"], w["hd"], w["S"]
    rng = np.random.default_rng(3001)
    blocks = [S.LlamaAttention(ctx, H, KV, hd, w["theta"], 1e-6,
                               q_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32),
                               k_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32), initial_capacity=T)
              for _ in range(w["layers_timed"])]
    g = torch.Generator(device=dev)
    g.manual_seed(3002)
    q = torch.randn(T, H * hd, device=dev, generator=g)
    k = torch.randn(T, KV * hd, device=dev, generator=g)
    v = torch.randn(T, KV * hd, device=dev, generator=g)
    out = torch.empty_like(q)
    best = None
    for rep in range(4):                       # first repetition is the warm-up
        for b in blocks:
            b.clear_cache()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for b in blocks:
            b.forward_cached_dev(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), T, stream_obj.cuda_stream)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / len(blocks)
        if rep > 0:
            best = ms if best is None else min(best, ms)
    # the tensor-core kernel alone: the library brackets its attention launch with events
    def kernel_ms(flags):
        ctx.timing_enable(True)
        for b in blocks:
            b.clear_cache()
        for b in blocks:
            b.forward_cached_dev(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), T, stream_obj.cuda_stream, flags)
        torch.cuda.synchronize()
        ms_, n_ = ctx.timing_read()
        ctx.timing_enable(False)
        return ms_ / max(n_, 1)
    kern_ms = kernel_ms(0)
    one_cta_ms = kernel_ms(S.F_TENSOR_1CTA)
    ctx.sync()
    for b in blocks:
        b.close()
    flops = 2.0 * hd * H * T * (T + 1)
    tfl = flops / (best / 1e3) / 1e12
    kern_tfl = flops / (kern_ms / 1e3) / 1e12
    try:
        bf16 = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
        peak, kind = bf16 / 2.0, "measured bf16 burst / 2 (TF32 issues at half the bf16 rate)"
    except Exception:
        peak, kind = 1590.0 / 2.0, "fallback bf16 / 2"
    return {"workload": w["name"], "ms_per_layer": best, "tflops": tfl, "layers_timed": len(blocks),
            "est_ms_all_layers": best * w["layers_total"],
            "note": "ms_per_layer and tflops cover both launches of a layer (norm/RoPE/append, then attention); "
                    "the roofline block is the attention kernel alone",
            "roofline": {"bound": "tensor", "kernel": "attn_prefill_pair_kernel (cluster of two CTAs, cta_group::2)",
                         "achieved": kern_tfl, "peak": peak,
                         "peak_kind": kind, "unit": "TFLOP/s", "frac": kern_tfl / peak, "kernel_ms": kern_ms,
                         "flops_per_launch": flops,
                         "single_cta_kernel_ms": one_cta_ms,
                         "single_cta_kernel_note": "attn_prefill_tc2_kernel on the same inputs (SHAINET_ATTN_F_TENSOR_1CTA)"}}


BATCHED_WL = dict(name="cfg4: Qwen3-8B attention, 64 sequences in lock step, context lengths log-uniform in [1k, 32k], fp32 KV cache, decode",
                  H=32, KV=8, hd=128, theta=1e6, batch=64, lo=1024, hi=32768, layers_total=36, steps=16)


def batched_block(S, ctx, dev, stream_obj, rank=0, world=1, dist=None, seqs=None, layers_resident=None, kv_format="f32"):
    """Batched ragged decode on the cfg4 shape: one launch per layer serves all 64 sequences (norm/RoPE/
    append and attention fused, two-level ticket merge).  Over several ranks the kv heads (and their
    query heads) are divided, every rank holds its heads of all 64 sequences, and the head outputs
    [64, q_dim / ranks] of a layer are all-gathered (NCCL, 1 MB per layer: a real exchange step, not
    latency-class) before o_proj would read them.  2 x ranks of the 36 layers are resident per rank
    (4.9 GB per layer over all ranks); the per-layer time scales to a step."""
    import torch
    w = BATCHED_WL
    H, KV, hd, B = w["H"], w["KV"], w["hd"], seqs or w["batch"]
    if KV % world:
        return None
    KVl, Hl = KV // world, H // world
    layers_timed = layers_resident or min(2 * world, 8)
    rng = np.random.default_rng(4001)
    lens = np.exp(rng.uniform(np.log(w["lo"]), np.log(w["hi"]), B)).astype(np.int64)
    steps, warm = w["steps"], 3
    qn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
    kn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
    layers = []
    for l in range(layers_timed):
        caches = []
        for b in range(B):
            a = S.LlamaAttention(ctx, Hl, KVl, hd, w["theta"], 1e-6, q_norm=qn, k_norm=kn,
                                 initial_capacity=int(lens[b]) + steps + warm + 8, kv_format=kv_format)
            a.cache.fill_normal(int(lens[b]), 4002 + 100000 * rank + 1000 * l + b)
            caches.append(a)
        layers.append(caches)
    g = torch.Generator(device=dev)
    g.manual_seed(4003 + rank)
    q = torch.randn(B, Hl * hd, device=dev, generator=g)
    k = torch.randn(B, KVl * hd, device=dev, generator=g)
    v = torch.randn(B, KVl * hd, device=dev, generator=g)
    out = torch.empty(layers_timed, B, Hl * hd, device=dev)
    gathered = torch.empty(layers_timed, world, B, Hl * hd, device=dev) if world > 1 else None
    scale = layers[0][0].scale
    handles = [[a.cache for a in caches] for caches in layers]

    def step():
        for l, hs in enumerate(handles):
            S.forward_batched_dev(ctx, hs, q.data_ptr(), k.data_ptr(), v.data_ptr(), out[l].data_ptr(), scale,
                                  stream_obj.cuda_stream)
            if world > 1:
                dist.all_gather_into_tensor(gathered[l].view(-1), out[l].view(-1))
    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ctx.sync()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_layer = ms / (steps * len(layers))
    mean_len = float(lens.sum()) + B * (warm + (steps + 1) / 2.0)
    es = 2 if kv_format == "bf16" else 4
    bytes_layer_rank = 2.0 * KVl * mean_len * hd * es + B * (2 * KVl * es + 2 * Hl * 4) * hd
    for caches in layers:
        for a in caches:
            a.close()
    check = batched_parity(S, ctx, w, rank, world, dev, stream_obj, dist, kv_format)
    peak, kind = measured_peak()
    gbs = bytes_layer_rank / (ms_layer / 1e3) / 1e9
    return {"workload": w["name"] if es == 4 else w["name"].replace("fp32 KV cache", "bfloat16 KV cache"), "sum_of_context_lengths": int(lens.sum()), "ms_per_layer": ms_layer,
            "tokens_per_s_36_layers": B / (ms_layer * w["layers_total"] / 1e3), "layers_timed": len(layers), "steps": steps,
            "sharding": (f"{world} rank(s) x {KVl} kv head(s) of every sequence"
                         + ("; head outputs all-gathered per layer (NCCL)" if world > 1 else "; no exchange")),
            "parity_check": check,
            "roofline": {"bound": "hbm", "kernel": "attn_decode_fused_kernel (batched)", "achieved": gbs, "peak": peak,
                         "peak_kind": kind, "unit": "GB/s per GPU", "frac": gbs / peak, "bytes_per_launch": bytes_layer_rank,
                         "note": "per GPU; the launch time includes the layer's all-gather when ranks > 1"}}


def batched_parity(S, ctx, w, rank, world, dev, stream_obj, dist, kv_format="f32"):
    """One checked lock-step step of the batched (and, over several ranks, kv-head-sharded and gathered)
    path: 5 short sequences with seeded caches against one CPU oracle per sequence, on rank 0."""
    import torch
    H, KV, hd = w["H"], w["KV"], w["hd"]
    KVl, Hl = KV // world, H // world
    rng = np.random.default_rng(4400)
    lens = [1, 40, 257, 600, 1031]
    B = len(lens)
    qn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
    kn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
    full = [(rng.standard_normal((KV, L, hd), dtype=np.float32), rng.standard_normal((KV, L, hd), dtype=np.float32)) for L in lens]
    q = rng.standard_normal((B, H * hd)).astype(np.float32)
    k = rng.standard_normal((B, KV * hd)).astype(np.float32)
    v = rng.standard_normal((B, KV * hd)).astype(np.float32)
    kvs = slice(rank * KVl, (rank + 1) * KVl)
    caches = []
    for kc, vc in full:
        a = S.LlamaAttention(ctx, Hl, KVl, hd, w["theta"], 1e-6, q_norm=qn, k_norm=kn, kv_format=kv_format)
        a.cache.import_(kc[kvs], vc[kvs])
        a.cache.reserve(kc.shape[1] + 2)
        caches.append(a)
    ql = q.reshape(B, H, hd)[:, rank * Hl:(rank + 1) * Hl].reshape(B, -1).copy()
    kl = k.reshape(B, KV, hd)[:, kvs].reshape(B, -1).copy()
    vl = v.reshape(B, KV, hd)[:, kvs].reshape(B, -1).copy()
    tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (ql, kl, vl))
    out = torch.zeros(B, Hl * hd, device=dev)
    S.forward_batched_dev(ctx, [a.cache for a in caches], tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(),
                          caches[0].scale, stream_obj.cuda_stream)
    if world > 1:
        gathered = torch.zeros(world, B, Hl * hd, device=dev)
        dist.all_gather_into_tensor(gathered.view(-1), out.view(-1))
        got = gathered.permute(1, 0, 2).reshape(B, H * hd).cpu().numpy()
    else:
        got = out.cpu().numpy()
    torch.cuda.synchronize()
    ctx.sync()
    for a in caches:
        a.close()
    if rank != 0:
        return None
    from oracle import oracle as O
    worst = 0.0
    for b, (kc, vc) in enumerate(full):
        o = O.OracleAttention(H, KV, hd, w["theta"], 1e-6, q_norm=qn, k_norm=kn,
                              kv_rounding="bf16" if kv_format == "bf16" else None)
        o.import_cache(kc, vc)
        ref = o.attend_cached(q[b:b + 1], k[b:b + 1], v[b:b + 1], threads=host_threads())
        worst = max(worst, float(np.abs(got[b:b + 1].astype(np.float64) - ref).max() / np.abs(ref).max()))
    return {"max_rel_err": worst, "tol": 1e-5, "ok": bool(worst <= 1e-5), "sequences": B, "ranks": world}


def short_context_block(S, ctx, dev, stream_obj, steps=128, warm=8):
    """The metric's ctx-4k point: BASELINE config 2's attention (LLaMA-3.2-1B: 16 layers, 32 query /
    8 kv heads, head_dim 64, batch 1, fp32 cache at ctx 4096).  The 16 layers' K/V (268 MB) are
    cycled, which is more than L2 holds, so every launch streams from HBM."""
    return decode_chain_block(S, ctx, dev, stream_obj, WORKLOADS["cfg2"], "f32", steps, warm)


def bf16_kv_block(S, ctx, dev, stream_obj):
    """The opt-in bfloat16 KV cache (no counterpart in the reference, whose rows are fp32; not the
    headline): the two decode points of the metric with rows rounded to bfloat16 as they are
    appended, fp32 arithmetic.  Algorithmic bytes count two bytes per cache element.  The ctx-4k
    point runs three copies of the 16 layers so that the cycled K/V (403 MB) exceed L2."""
    out = []
    batched = batched_block(S, ctx, dev, stream_obj, kv_format="bf16")
    for key, steps, copies in (("cfg5", 24, 1), ("cfg2", 64, 3)):
        wl = dict(WORKLOADS[key])
        wl["name"] = wl["name"].replace("fp32 KV cache", "bfloat16 KV cache")
        res = decode_chain_block(S, ctx, dev, stream_obj, wl, "bf16", steps, 6, copies)
        res["parity_check"] = format_parity(S, ctx, wl, "bf16")
        out.append(res)
    out.append(batched)
    return out


def format_parity(S, ctx, wl, kv_format, ctx_len=2053):
    """One checked decode step over a cache of the given element format against the CPU oracle with the
    same row rounding, at a context the oracle finishes in a moment."""
    from oracle import oracle as O
    H, KV, hd = wl["H"], wl["KV"], wl["hd"]
    rng = np.random.default_rng(611)
    kw = {}
    if wl["qk_norm"]:
        kw = dict(q_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32),
                  k_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32))
    o = O.OracleAttention(H, KV, hd, wl["theta"], 1e-6, kv_rounding="bf16" if kv_format == "bf16" else None, **kw)
    g = S.LlamaAttention(ctx, H, KV, hd, wl["theta"], 1e-6, kv_format=kv_format, **kw)
    kc = rng.standard_normal((KV, ctx_len, hd), dtype=np.float32)
    vc = rng.standard_normal((KV, ctx_len, hd), dtype=np.float32)
    o.import_cache(kc, vc)
    g.cache.import_(kc, vc)
    q, k, v = (rng.standard_normal((1, n), dtype=np.float32) for n in (H * hd, KV * hd, KV * hd))
    ref = o.attend_cached(q, k, v, threads=host_threads())
    got = g.forward_cached(q, k, v)
    g.close()
    err = float(np.abs(got.astype(np.float64) - ref).max() / np.abs(ref).max())
    return {"max_rel_err": err, "tol": 1e-5, "ok": bool(err <= 1e-5), "ctx": ctx_len,
            "what": "one decode step against the CPU oracle whose cache rows are rounded the same way"}


def decode_chain_block(S, ctx, dev, stream_obj, wl, kv_format, steps, warm, copies=1):
    """Batch-1 decode attention of a whole model's layers (times `copies`), one fused launch per
    layer-step, timed with CUDA events on the launching stream."""
    import torch
    H, KV, hd, layers, L = wl["H"], wl["KV"], wl["hd"], wl["layers"] * copies, wl["ctx"]
    es = 2 if kv_format == "bf16" else 4
    rng = np.random.default_rng(2100)
    kw = {}
    if wl["qk_norm"]:
        kw = dict(q_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32),
                  k_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32))
    blocks = []
    for l in range(layers):
        b = S.LlamaAttention(ctx, H, KV, hd, wl["theta"], 1e-5, initial_capacity=L + steps + warm + 8,
                             kv_format=kv_format, **kw)
        b.cache.fill_normal(L, 2101 + l)
        blocks.append(b)
    g = torch.Generator(device=dev)
    g.manual_seed(2102)
    q = torch.randn(layers, H * hd, device=dev, generator=g)
    k = torch.randn(layers, KV * hd, device=dev, generator=g)
    v = torch.randn(layers, KV * hd, device=dev, generator=g)
    out = torch.empty_like(q)
    fwd = ctx.L.shainet_attn_forward_dev
    vp = C.c_void_p
    call = [(ctx.h, b.cache.h, vp(q[l].data_ptr()), vp(k[l].data_ptr()), vp(v[l].data_ptr()), vp(out[l].data_ptr()), 1,
             C.c_float(b.scale), 0, vp(stream_obj.cuda_stream)) for l, b in enumerate(blocks)]

    def run(n):
        for _ in range(n):
            for a in call:
                rc = fwd(*a)
                if rc:
                    S.check(rc)
    run(warm)
    torch.cuda.synchronize()
    for b in blocks:
        b.cache.truncate(L)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(steps)
    e1.record()
    torch.cuda.synchronize()
    ctx.sync()
    ms = e0.elapsed_time(e1)
    for b in blocks:
        b.close()
    peak, kind = measured_peak()
    bytes_launch = decode_bytes(wl, L + (steps + 1) / 2.0, elem_bytes=es)
    us = ms * 1e3 / (steps * layers)
    gbs = bytes_launch / (us * 1e-6) / 1e9
    ms /= copies   # a step of the model is one pass over its own layers
    return {"workload": wl["name"], "tokens_per_s": steps / (ms / 1e3), "ms_per_step": ms / steps, "steps": steps,
            "roofline": {"bound": "hbm", "kernel": "attn_decode_fused_kernel", "achieved": gbs, "peak": peak,
                         "peak_kind": kind, "unit": "GB/s", "frac": gbs / peak, "bytes_per_launch": bytes_launch,
                         "avg_launch_us": us, "launches_timed": steps * layers}}


def gemv_block(S, ctx, dev, stream_obj):
    """Q8_0 GEMV (one activation row) at the projection shapes of the LLaMA-3.2-1B block: bytes = one per weight
    plus four per 32-weight scale, over the time of a launch in a chain of launches on one stream (each launch
    waits for the one before it, as in decode).  Every shape cycles over enough distinct weights to exceed L2."""
    import torch
    g = torch.Generator(device=dev)
    g.manual_seed(2401)
    peak, kind = measured_peak()
    out = []
    for name, K, N in (("q_proj / o_proj", 2048, 2048), ("k_proj / v_proj", 2048, 512), ("q|k|v stacked", 2048, 3072),
                       ("gate_proj / up_proj", 2048, 8192), ("down_proj", 8192, 2048)):
        per = K * N + 4 * N * (K // 32)
        count = max(4, int(400e6 // per))
        keep, ws = [], []
        for _ in range(count):
            q = torch.randint(-127, 128, (N, K), device=dev, dtype=torch.int8, generator=g)
            sc = (0.02 / 127.0) * (0.5 + torch.rand(N, K // 32, device=dev, generator=g))
            keep.extend([q, sc])
            ws.append(S.Q8Weight.wrap(ctx, q.data_ptr(), sc.data_ptr(), K, N))
        x = torch.randn(1, K, device=dev, generator=g)
        y = torch.empty(1, N, device=dev)
        calls = []
        gemv = ctx.L.shainet_attn_q8_gemv_dev
        vp = C.c_void_p
        for i in range(count):
            calls.append((ctx.h, ws[i].h, vp(x.data_ptr()), vp(y.data_ptr()), 1, vp(stream_obj.cuda_stream)))
        reps = 6

        def run(n):
            for _ in range(n):
                for a in calls:
                    rc = gemv(*a)
                    if rc:
                        S.check(rc)
        run(1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run(reps)
        e1.record()
        torch.cuda.synchronize()
        ctx.sync()
        us = e0.elapsed_time(e1) * 1e3 / (reps * count)
        single = K * N + 4 * N * (K // 32)
        gbs = single / (us * 1e-6) / 1e9
        out.append({"shape": name, "K": K, "N": N,
                    "bytes_per_launch": single, "us_per_launch": us, "gbs": gbs, "frac": gbs / peak, "weights_cycled": count})
        for w in ws:
            w.close()
        del keep
    return {"kernel": "q8_gemv_ring_kernel (one row)", "peak": peak, "peak_kind": kind, "unit": "GB/s", "shapes": out,
            "note": "launches are chained on one stream, each waiting for its predecessor; us_per_launch therefore "
                    "includes the dependent-launch latency that dominates at these sizes (1.3 to 19 MB per launch)"}


def model_decode_block(S, ctx, dev, steps=96, warm=8):
    """BASELINE config 2 as a whole model on the device: 16 LLaMA-3.2-1B-shaped blocks (hidden 2048, 32/8
    heads, head_dim 64, FFN 8192), vocabulary 128256, every projection / FFN / lm_head weight Q8_0, fp32
    KV cache at ctx 4096, greedy decode.  One call generates `steps` tokens; the only host traffic is the
    first token id in and the generated ids out, so the wall clock of the call is the end-to-end figure.
    Weights are random int8 with random scales created on the device (distinct memory per layer, 1.4 GB in
    all, far more than L2 holds); bytes per token = all weights and scales once + the K/V of every layer."""
    import torch
    wl = WORKLOADS["cfg2"]
    H, KV, hd, layers, L = wl["H"], wl["KV"], wl["hd"], wl["layers"], wl["ctx"]
    d, ffn, vocab, eps = 2048, 8192, 128256, 1e-5
    g = torch.Generator(device=dev)
    g.manual_seed(2201)
    keep, weight_bytes = [], 0

    def q8(K, N):
        nonlocal weight_bytes
        q = torch.randint(-127, 128, (N, K), device=dev, dtype=torch.int8, generator=g)
        sc = (0.02 / 127.0) * (0.5 + torch.rand(N, K // 32, device=dev, generator=g))
        keep.extend([q, sc])
        weight_bytes += q.numel() + 4 * sc.numel()
        return S.Q8Weight.wrap(ctx, q.data_ptr(), sc.data_ptr(), K, N)

    ones = np.ones(d, np.float32)
    blocks, attns, weights = [], [], []
    for l in range(layers):
        a = S.LlamaAttention(ctx, H, KV, hd, wl["theta"], eps, initial_capacity=L + steps + warm + 8)
        a.cache.fill_normal(L, 2301 + l)
        w = dict(wq=q8(d, H * hd), wk=q8(d, KV * hd), wv=q8(d, KV * hd), wo=q8(H * hd, d), gate=q8(d, ffn), up=q8(d, ffn),
                 down=q8(ffn, d))
        blocks.append(S.LlamaBlock(ctx, a, d, eps, ones, w["wq"], w["wk"], w["wv"], w["wo"], ones, w["gate"], w["up"], w["down"]))
        attns.append(a)
        weights.extend(w.values())
    head = q8(d, vocab)
    weights.append(head)
    emb = (0.02 * np.random.default_rng(2202).standard_normal((vocab, d), dtype=np.float32))
    dec = S.Decoder(ctx, blocks, emb, ones, head, None, eps)
    del emb
    dec.generate([1], warm)
    for a in attns:
        a.cache.truncate(L)
    t0 = time.perf_counter()
    toks = dec.generate([1], steps)
    wall = time.perf_counter() - t0
    dec.close()
    for b in blocks:
        b.close()
    for a in attns:
        a.close()
    for w in weights:
        w.close()
    kv_bytes = layers * decode_bytes(wl, L + (steps + 1) / 2.0)
    per_token = weight_bytes + kv_bytes + d * 4
    peak, kind = measured_peak()
    gbs = per_token * steps / wall / 1e9
    return {"workload": "cfg2: LLaMA-3.2-1B-shaped decoder, 16 layers, vocabulary 128256, Q8_0 weights, fp32 KV cache ctx 4096, "
                        "greedy decode on the device (shainet_attn_decoder_generate)",
            "tokens_per_s": steps / wall, "ms_per_token": wall / steps * 1e3, "steps": steps,
            "distinct_tokens": int(len(set(toks.tolist()))),
            "h2d_bytes_per_call": 4, "d2h_bytes_per_call": 4 * steps, "launches_per_token": 5 * layers + 3,
            "timing": "wall clock of one blocking generate call (prompt of one token, then steps - 1 device-fed steps)",
            "roofline": {"bound": "hbm", "kernel": "q8_gemv_kernel + attn_decode_fused_kernel chain", "achieved": gbs, "peak": peak,
                         "peak_kind": kind, "unit": "GB/s", "frac": gbs / peak, "bytes_per_token": per_token,
                         "weight_bytes": weight_bytes, "kv_bytes": kv_bytes}}


PARITY_TOL = 1e-5


def parity_check(S, ctx, wl, sp, rank, world, dev, stream, dist, peer, comm_slot_floats, epoch):
    """One checked layer-step on the very path the timed region used (same entry points, same sharding,
    same exchange): every rank imports its part of one seeded cache of 2053 positions, attends for one
    new token, and rank 0 compares the gathered (and, for a split sequence, merged) head outputs of all
    ranks with the CPU oracle's unsharded result.  Returns the dictionary for the JSON line."""
    import torch
    H, KV, hd = wl["H"], wl["KV"], wl["hd"]
    Hl, KVl = sp.head_count, sp.kv_count
    split = sp.seq_parts > 1
    Lc = 2053
    rng = np.random.default_rng(777)          # the same stream on every rank: identical full inputs
    kw = {}
    if wl["qk_norm"]:
        kw = dict(q_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32),
                  k_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32))
    kc = rng.standard_normal((KV, Lc, hd), dtype=np.float32)
    vc = rng.standard_normal((KV, Lc, hd), dtype=np.float32)
    q = rng.standard_normal((1, H * hd)).astype(np.float32)
    k = rng.standard_normal((1, KV * hd)).astype(np.float32)
    v = rng.standard_normal((1, KV * hd)).astype(np.float32)
    g = S.LlamaAttention(ctx, Hl, KVl, hd, wl["theta"], 1e-6, initial_capacity=Lc + 8, **kw)
    kvs = slice(sp.kv_begin, sp.kv_begin + KVl)
    g.cache.import_(kc[kvs, sp.seq_part::sp.seq_parts], vc[kvs, sp.seq_part::sp.seq_parts])
    ql = q.reshape(1, H, hd)[:, sp.head_begin:sp.head_begin + Hl].reshape(1, -1).copy()
    kl = k.reshape(1, KV, hd)[:, kvs].reshape(1, -1).copy()
    vl = v.reshape(1, KV, hd)[:, kvs].reshape(1, -1).copy()
    tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (ql, kl, vl))
    pay = Hl * hd + (Hl if split else 0)
    out = torch.zeros(pay, device=dev)
    full = torch.zeros(H * hd, device=dev)
    pos, own = Lc, sp.owns_position(Lc)
    if world > 1:
        dist.barrier()
    if world == 1:
        g.forward_cached_dev(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), full.data_ptr(), 1, stream)
    elif peer and split:
        g.forward_cached_dev_exchange_merge(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), pos, own, 0,
                                            sp.seq_parts, epoch, full.data_ptr(), stream)
    elif peer:
        g.forward_cached_dev_exchange(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), pos, own,
                                      rank * pay, -1, 0, world * pay, epoch, stream)
        host = np.empty(world * pay, np.float32)
        ctx.comm_read(0, host, stream)
    else:
        gathered = torch.empty(world, pay, device=dev)
        if split:
            ctx.set_lse_out(out[Hl * hd:].data_ptr())
        g.forward_cached_dev_at(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), pos, own, stream)
        ctx.set_lse_out(None)
        dist.all_gather_into_tensor(gathered.view(-1), out)
        if split:
            ctx.merge_parts(gathered.data_ptr(), world, sp.seq_parts, Hl, hd, full.data_ptr(), stream)
        else:
            full = gathered.view(-1)
    torch.cuda.synchronize()
    ctx.sync()
    got = host if (peer and not split and world > 1) else full.cpu().numpy()
    g.close()
    res = None
    if rank == 0:
        from oracle import oracle as O
        o = O.OracleAttention(H, KV, hd, wl["theta"], 1e-6, **kw)
        o.import_cache(kc, vc)
        ref = o.attend_cached(q, k, v, threads=host_threads())[0]
        err = float(np.abs(got.astype(np.float64) - ref).max() / np.abs(ref).max())
        res = {"max_rel_err": err, "tol": PARITY_TOL, "ok": bool(err <= PARITY_TOL), "ctx": Lc, "ranks": world,
               "what": "one layer-step of this run's path (sharding and exchange included) against the CPU oracle's "
                       "unsharded attention on the same seeded cache"}
    if world > 1:
        dist.barrier()
    return res


def run_one_block(args):
    """--only NAME: one of the secondary blocks alone, printed as its own JSON object (profiling and
    quick measurements; the driver's line is the default run)."""
    import torch
    import shainet_b200 as S
    from shainet_b200 import build
    build.build()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    ctx = S.AttnContext(0)
    tstream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(tstream)
    if args.only == "gemv":
        res = gemv_block(S, ctx, dev, tstream)
    elif args.only == "model":
        res = model_decode_block(S, ctx, dev, steps=args.steps if args.steps != 256 else 96)
    elif args.only == "ctx4k":
        res = short_context_block(S, ctx, dev, tstream)
    elif args.only == "bf16kv":
        res = bf16_kv_block(S, ctx, dev, tstream)
    elif args.only == "batched":
        res = batched_block(S, ctx, dev, tstream, seqs=args.batched_seqs, layers_resident=args.batched_layers,
                            kv_format=args.kv_format)
    else:
        res = prefill_block(S, ctx, dev, tstream)
    ctx.close()
    print(json.dumps({args.only: res}), flush=True)


def run_ours(args, wl, rank, world, local_rank):
    import torch
    import shainet_b200 as S
    from shainet_b200 import build
    build.build()

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
    H, KV, hd, layers, ctx_len = wl["H"], wl["KV"], wl["hd"], wl["layers"], wl["ctx"]
    # kv-head groups over the ranks; with more ranks than kv heads the ranks of a
    # group also split the positions round-robin (shainet_b200/sharding.py)
    sp = S.sharding.plan(world, rank, H, KV)
    KVl, Hl = sp.kv_count, sp.head_count
    qd, kd = Hl * hd, KVl * hd
    local_ctx = sp.local_rows(ctx_len)
    K, W = args.steps, args.warmup
    K_roof = min(K, 32)
    K_e2e, W_e2e = min(K, 64), 3

    rng = np.random.default_rng(5000 + rank)
    ctx = S.AttnContext(local_rank)
    cap = local_ctx + max(K, W, K_roof, K_e2e + W_e2e) + 8
    blocks = []
    for l in range(layers):
        kw = {}
        if wl["qk_norm"]:
            kw = dict(q_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32),
                      k_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32))
        b = S.LlamaAttention(ctx, Hl, KVl, hd, wl["theta"], 1e-6, initial_capacity=cap, **kw)
        b.cache.fill_normal(local_ctx, 5001 + 1000 * rank + l)
        blocks.append(b)

    NV = 4  # input variants cycled over steps
    g = torch.Generator(device=dev)
    g.manual_seed(5002 + rank)
    q_d = torch.randn(NV, layers, qd, device=dev, generator=g)
    k_d = torch.randn(NV, layers, kd, device=dev, generator=g)
    v_d = torch.randn(NV, layers, kd, device=dev, generator=g)
    split = sp.seq_parts > 1
    pay = qd + (Hl if split else 0)        # a rank's contribution per layer: outputs (+ log-sum-exp when the sequence is split)
    out_d = torch.empty(layers, pay, device=dev)
    # Several ranks: every rank's fused kernel stores its head rows straight into all
    # ranks' exchange buffers over NVLink (layout [layer][rank][pay]) as {value, epoch}
    # words; a small kernel per layer waits for the words of all ranks and unpacks them.  --nccl-gather keeps the
    # torch.distributed all-gather instead (also used when rows are not 16-byte multiples).
    peer = world > 1 and pay % 4 == 0 and not args.nccl_gather
    gathered = torch.empty(layers, world, pay, device=dev) if world > 1 and not peer else None
    comm_base = None
    if peer:
        mine = ctx.comm_create(layers * world * pay)
        handles = [None] * world
        dist.all_gather_object(handles, mine)
        ctx.comm_open(handles, rank)
        comm_base = ctx.comm_data_ptr()
        dist.barrier()
    epoch = [0]
    full_d = torch.empty(layers, H * hd, device=dev) if split else None
    # Everything timed runs on one explicit (non-default) stream: the library is
    # handed its handle, and the CUDA events are recorded on it.
    tstream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(tstream)
    stream = tstream.cuda_stream
    assert stream != 0
    esz = q_d.element_size()
    torch.cuda.synchronize()

    def reset():
        for b in blocks:
            b.cache.truncate(local_ctx)

    # Pre-built argument lists keep the host cost of a launch to one foreign call.
    fwd_dev = ctx.L.shainet_attn_forward_dev
    vp = C.c_void_p
    def build_args(flags):
        return [[(ctx.h, b.cache.h, vp(q_d[vi, l].data_ptr()), vp(k_d[vi, l].data_ptr()), vp(v_d[vi, l].data_ptr()),
                  vp(out_d[l].data_ptr()), 1, C.c_float(b.scale), flags, vp(stream)) for l, b in enumerate(blocks)]
                for vi in range(NV)]
    dev_args = build_args(0)

    fwd_at = ctx.L.shainet_attn_forward_dev_at
    set_lse = ctx.L.shainet_attn_ctx_set_lse_out
    merge = ctx.L.shainet_attn_merge_parts
    lse_ptrs = [vp(out_d[l, qd:].data_ptr()) for l in range(layers)] if split else None
    if split:
        gath_ptrs = [vp(comm_base + l * world * pay * 4) if peer else vp(gathered[l].data_ptr()) for l in range(layers)]
    fwd_x = ctx.L.shainet_attn_forward_dev_exchange
    fwd_xm = ctx.L.shainet_attn_forward_dev_exchange_merge
    out_offs = [(l * world + rank) * pay for l in range(layers)]
    full_ptrs = [vp(full_d[l].data_ptr()) for l in range(layers)] if split else None

    def step(i, all_args=None):
        args = (all_args or dev_args)[i % NV]
        epoch[0] += 1
        ep = epoch[0]
        pos = ctx_len + i                   # the token's position; with a split sequence its k/v row goes to one rank of the group
        own = 1 if sp.owns_position(pos) else 0
        if peer and split:
            for l in range(layers):                 # deliver, wait for all ranks and merge the sequence parts: one call
                a = args[l]
                rc = fwd_xm(a[0], a[1], a[2], a[3], a[4], a[5], pos, own, a[7], a[8], l * world * pay, sp.seq_parts, ep,
                            full_ptrs[l], a[9])
                if rc:
                    S.check(rc)
            return
        if peer:
            for l in range(layers):
                a = args[l]
                rc = fwd_x(a[0], a[1], a[2], a[3], a[4], a[5], pos, own, a[7], a[8], out_offs[l],
                           out_offs[l] + qd if split else -1, l * world * pay, world * pay, ep, a[9])   # head outputs of all ranks, before o_proj
                if rc:
                    S.check(rc)
                if split:
                    rc = merge(ctx.h, gath_ptrs[l], world, sp.seq_parts, Hl, hd, full_ptrs[l], a[9])
                    if rc:
                        S.check(rc)
            return
        if not split:
            for l in range(layers):
                rc = fwd_dev(*args[l])
                if rc:
                    S.check(rc)
                if world > 1:
                    dist.all_gather_into_tensor(gathered[l].view(-1), out_d[l])
            return
        for l in range(layers):
            a = args[l]
            set_lse(ctx.h, lse_ptrs[l])
            rc = fwd_at(a[0], a[1], a[2], a[3], a[4], a[5], pos, own, a[7], a[8], a[9])
            if rc:
                S.check(rc)
            dist.all_gather_into_tensor(gathered[l].view(-1), out_d[l])
            rc = merge(ctx.h, gath_ptrs[l], world, sp.seq_parts, Hl, hd, full_ptrs[l], a[9])
            if rc:
                S.check(rc)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    for i in range(max(W, 3)):
        step(i)
    barrier()
    sampler.start()
    reset()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    t_enq = time.perf_counter()
    for i in range(K):
        step(i)
    t_enq = time.perf_counter() - t_enq   # host time to enqueue the region (must stay below the device time)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    ctx.sync()
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    # ---- host cost of a layer call, measured on a burst short enough not to fill the launch queue ----
    reset()
    barrier()
    t_burst = time.perf_counter()
    for i in range(4):
        step(i)
    host_call_us = (time.perf_counter() - t_burst) * 1e6 / (4 * layers)
    barrier()

    # ---- same region with F_INPUTS_READY: this bench's inputs are resident long before the
    # launches, so consecutive layers may overlap fully (reported beside the headline) ----
    ready_args = build_args(S.F_INPUTS_READY)
    reset()
    barrier()
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for i in range(K):
        step(i, ready_args)
    r1.record()
    barrier()
    ms_ready = r0.elapsed_time(r1)

    # ---- isolated launches: each kernel bracketed by events inside the library (no overlap) ----
    reset()
    ctx.timing_enable(True)
    for i in range(K_roof):
        step(i)
    barrier()
    kernel_ms, launches = ctx.timing_read()
    ctx.timing_enable(False)
    clocks = sampler.stop()

    # ---- end to end: host-pointer C-ABI entry, pinned host inputs, blocking ----
    reset()
    hq = torch.randn(NV, layers, qd).pin_memory()
    hk = torch.randn(NV, layers, kd).pin_memory()
    hv = torch.randn(NV, layers, kd).pin_memory()
    ho = torch.empty(layers, qd).pin_memory()
    fwd_host = ctx.L.shainet_attn_forward_host
    FP = C.POINTER(C.c_float)

    ho_full = torch.empty(layers, (H * hd) if split else (world * qd), dtype=torch.float32).pin_memory() if world > 1 else None

    # the argument lists of the per-layer calls, built once: the pointers into the pinned buffers do not change, and
    # building them (tensor views, casts) per call would put several microseconds of Python into every layer
    host_calls = None
    if world == 1:
        host_calls = [[(ctx.h, b.cache.h, C.cast(hq[vi, l].data_ptr(), FP), C.cast(hk[vi, l].data_ptr(), FP),
                        C.cast(hv[vi, l].data_ptr(), FP), C.cast(ho[l].data_ptr(), FP), 1, C.c_float(b.scale), 0)
                       for l, b in enumerate(blocks)] for vi in range(NV)]

    def host_step(i):
        vi = i % NV
        if world == 1:
            for call in host_calls[vi]:
                rc = fwd_host(*call)
                if rc:
                    S.check(rc)
            return
        # several ranks: this step's inputs come from pinned host memory, the gathered
        # (and merged) head outputs of every layer go back to pinned host memory
        q_d[vi].copy_(hq[vi], non_blocking=True)
        k_d[vi].copy_(hk[vi], non_blocking=True)
        v_d[vi].copy_(hv[vi], non_blocking=True)
        step(i)
        if peer and not split:
            rc = ctx.L.shainet_attn_comm_read(ctx.h, 0, C.cast(ho_full.data_ptr(), FP), ho_full.numel(), vp(stream))
            if rc:
                S.check(rc)
        else:
            ho_full.copy_((full_d if split else gathered.view(layers, -1)), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    for i in range(W_e2e):
        host_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(K_e2e):
        host_step(W_e2e + i)
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    prefill = batched = short_ctx = None
    if world == 1 and not args.no_prefill:
        prefill = prefill_block(S, ctx, dev, tstream)
    if not args.no_prefill:
        batched = batched_block(S, ctx, dev, tstream, rank, world, dist)
    model = gemv = bf16kv = None
    if world == 1 and not args.no_prefill and args.workload != "cfg2":
        short_ctx = short_context_block(S, ctx, dev, tstream)
        bf16kv = bf16_kv_block(S, ctx, dev, tstream)
        model = model_decode_block(S, ctx, dev)
        gemv = gemv_block(S, ctx, dev, tstream)
    parity = parity_check(S, ctx, wl, sp, rank, world, dev, stream, dist, peer, layers * world * pay, epoch[0] + 1)

    if rank == 0:
        peak, peak_kind = measured_peak()
        # One fused kernel per layer-step: its average duration over the timed
        # region is the region's device time divided by the launches in it
        # (consecutive launches overlap through programmatic stream
        # serialization, so a per-launch event bracket would serialise them).
        bytes_per_launch = decode_bytes(wl, local_ctx + (K + 1) / (2.0 * sp.seq_parts), KVl)
        avg_kernel_s = ms / 1e3 / (K * layers)
        achieved = bytes_per_launch / avg_kernel_s / 1e9
        isolated_us = kernel_ms * 1e3 / max(launches, 1)
        line = {
            "metric": "decode_attn_tokens_per_s", "value": K / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["name"], "layers": layers, "num_heads": H, "num_kv_heads": KV, "head_dim": hd,
                       "ctx": ctx_len, "sharding": f"{sp.groups} kv-head group(s) x {sp.seq_parts} sequence part(s) over {world} rank(s); " + ("no exchange" if world == 1 else ("head outputs stored into every rank's buffer by the decode kernel (8-byte value+epoch peer stores over NVLink), one wait-and-unpack kernel per layer" if peer else "torch.distributed all-gather of head outputs per layer")),
                       "l2": "working set per step (all layers' K/V) is far larger than L2; no flush needed",
                       "host_enqueue_ms_per_step": t_enq * 1e3 / K, "host_us_per_layer_call": host_call_us,
                       "hbm_gbs_whole_step_per_gpu": bytes_per_launch * layers / (ms / K / 1e3) / 1e9},
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "attn_decode_fused_kernel", "achieved": achieved,
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": bytes_per_launch * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE if args.workload == "cfg5" and world == 1 else None,
                         "traffic_note": "ncu dram read+write bytes of one launch at L=32770, scaled by the rows of this run",
                         "bytes_per_launch": bytes_per_launch,
                         "avg_launch_us": avg_kernel_s * 1e6, "launches_timed": K * layers,
                         "isolated_launch_us": isolated_us, "isolated_launches": launches},
            "inputs_ready_mode": {"value": K / (ms_ready / 1e3), "unit": "tokens/s", "avg_launch_us": ms_ready * 1e3 / (K * layers),
                                  "gbs": bytes_per_launch / (ms_ready / 1e3 / (K * layers)) / 1e9,
                                  "note": "same region with SHAINET_ATTN_F_INPUTS_READY (q/k/v not produced by the previous launch)"},
            "e2e": {"value": K_e2e / e2e_s, "unit": "tokens/s", "steps": K_e2e,
                    "h2d_bytes_per_step": layers * (qd + 2 * kd) * esz,
                    "d2h_bytes_per_step": layers * (qd if world == 1 else H * hd) * esz,
                    "method": ("one blocking shainet_attn_forward_host call per layer: pinned host q/k/v in, host "
                               "output row back, stream synchronised every layer (the reference block's call pattern)"
                               if world == 1 else
                               "per step: three bulk copies of all layers' q/k/v from pinned host memory, the layers "
                               "queued asynchronously (forward_dev_exchange), one copy of all layers' gathered head "
                               "outputs back, one synchronisation; not comparable with the per-layer blocking method "
                               "used at one GPU")},
            "parity_check": parity,
            "gpu_launches": layers * K * (2 if peer else 1) + (layers * K if split and not peer else 0),
        }
        if prefill is not None:
            line["prefill"] = prefill
        if batched is not None:
            line["batched_decode"] = batched
        if short_ctx is not None:
            line["decode_ctx4k"] = short_ctx
        if bf16kv is not None:
            line["decode_bf16_kv"] = bf16kv
        if model is not None:
            line["decode_model_cfg2"] = model
        if gemv is not None:
            line["q8_gemv"] = gemv
        if world == 1 and not args.no_cpu_baseline:
            threads = host_threads()
            cpu_port_rate(wl, threads, 1, 1)
            per_step = cpu_port_rate(wl, threads, 2, 4)
            spt = float(np.mean(per_step)) * layers / 2
            one = cpu_port_rate(wl, 1, 1, 1)
            line["cpu_baseline"] = {"value": 1.0 / spt, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": f"4 decode steps x 2 of {layers} layers at ctx {ctx_len}, scaled to all "
                                              "layers; OpenMP over (query head, row block) work items",
                                    "single_thread_value": 1.0 / (float(one[0]) * layers)}
        print(json.dumps(line), flush=True)
    for b in blocks:
        b.close()
    ctx.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0 and not parity["ok"]:
        sys.exit(f"parity check failed: max relative error {parity['max_rel_err']:.3e} > {PARITY_TOL}")
    if rank == 0 and batched is not None and not batched["parity_check"]["ok"]:
        sys.exit(f"batched parity check failed: max relative error {batched['parity_check']['max_rel_err']:.3e}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg5", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (debugging / profiling)")
    ap.add_argument("--ctx", type=int, default=None, help="override the context length (debugging / profiling)")
    ap.add_argument("--heads", type=str, default=None,
                    help="override 'query_heads,kv_heads' (debugging: e.g. 8,1 on 2 ranks runs the sequence-split path)")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="several ranks: gather head outputs with torch.distributed instead of the kernel's peer stores")
    ap.add_argument("--only", default=None, choices=["model", "gemv", "ctx4k", "bf16kv", "batched", "prefill"],
                    help="run one secondary block alone on one GPU and print its JSON object")
    ap.add_argument("--batched-seqs", type=int, default=None, help="--only batched: sequences in the batch (profiling: a small resident case)")
    ap.add_argument("--kv-format", default="f32", choices=["f32", "bf16"], help="--only batched: element format of the caches")
    ap.add_argument("--batched-layers", type=int, default=None, help="--only batched: resident layers")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill (cfg3 shape) block of the JSON line")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload])
    if args.layers:
        wl["layers"] = args.layers
        wl["name"] += f" [layers={args.layers}]"
    if args.ctx:
        wl["ctx"] = args.ctx
        wl["name"] += f" [ctx={args.ctx}]"
    if args.heads:
        wl["H"], wl["KV"] = (int(x) for x in args.heads.split(","))
        wl["name"] += f" [heads={args.heads}]"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.only:
        run_one_block(args)
    elif args.impl == "reference":
        run_reference(args, wl, rank, world)
    else:
        run_ours(args, wl, rank, world, local_rank)


if __name__ == "__main__":
    main()
