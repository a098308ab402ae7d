#!/usr/bin/env python
"""Benchmark of the pruned decoder layer (Llama-3-70B-shaped, 16384-token prefill).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: hidden 8192, intermediate 28672 as 224 groups of 128 channels (half of them kept
per token), 64 query / 8 KV heads of dimension 128 (6 of 8 head groups kept per token),
16384 tokens, bf16, seeded synthetic tensors.  One step = the whole layer from the residual
stream: attention router + decision + RMSNorm (one kernel), routed Q projection, K/V
projections, rotary embedding, head-group-routed causal attention, routed output projection
(+ residual), FFN router + decision + RMSNorm, dynamic-width SwiGLU FFN (+ residual).  With
N > 1 the layer is tensor-parallel by KV-head groups and FFN channel groups; the partial sums
of the output and down projections are added by the fused row-parallel sum (stores into the
owning rank's memory over NVLink, then a reduce + gather kernel) -- total work is fixed
(strong scaling).

Prints ONE JSON line on rank 0.  Keys beyond the common contract:
  roofline      dominant kernel (fused gate/up GEMM) against the measured bf16 peak
  kernels       per-phase mean time inside the timed region (CUDA events)
  dense         the same layer without routing (cuBLAS, SDPA, NCCL all-reduce), same run
  parity        sampled token rows of the step's output against the CPU oracle
  configs       N = 1: sub-records of the FFN-prefill, attention-prefill and decode-step
                configurations (time, rate, roofline fraction, parity on sampled rows)
  cpu_baseline  the reference's CPU formulation (dense, then mask) on the host cores
  e2e           the same metric with host buffers: pinned H2D of x and D2H of the output
                inside the timed region, double buffered; every rank moves its own rows
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "llm-pruning_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "prefill_tokens_per_s_pruned_decoder_layer"
UNIT = "tokens/s"
TOL = 2e-2
CPU_SAMPLE_STRIDE = 8          # the CPU legs time every 8th token row of the sequence


def measured_peaks():
    """(sustained bf16 TFLOP/s, burst bf16 TFLOP/s, HBM GB/s, source)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return (d.get("bf16_tflops_sustained", 1425.8), d.get("bf16_tflops", 1668.9),
                d.get("hbm_gbs", 6449.1), "measured")
    return 1400.0, 1590.0, 6650.0, "fallback"


def recorded_traffic(shape, world: int):
    """DRAM bytes of one full-size launch of the dominant kernel as ncu measured them (read +
    write), from the summary under profiles/; None for any other shape or split."""
    if world != 1 or shape.tokens != 16384:
        return None
    path = os.path.join(ROOT, "profiles", "gemm_mn_pair_config5_counters.md")
    try:
        with open(path) as f:
            for line in f:
                if line.startswith("traffic_bytes_per_launch_config5_16384_tokens:"):
                    return float(line.split(":", 1)[1])
    except OSError:
        pass
    return None


def make_config(shape, world: int, args) -> dict:
    """The ``config`` object of the JSON line; the same for both arms at a given N."""
    if world == 1:
        par = "single GPU"
    else:
        par = (f"tp{world} by KV-head groups ({shape.attn_groups // world} per rank) and FFN channel "
               f"groups ({shape.ffn_groups // world} per rank); row-parallel sums of the o and down "
               f"projections: {args.sum}")
    return {"workload": shape.name, "parallelism": par,
            "routing": "two-stage token routers with argmax decisions, biased to the stated keep fractions",
            "l2": "per step the layer streams 2.4 GB of weights and > 1 GB of activations: larger than L2",
            "seed": 17}


# ------------------------------------------------------------------ clocks sampling

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.proc = None
        self.path = os.path.join("/tmp", f"dpk_clocks_{os.getpid()}.csv")
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            ident = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            ident = str(device_index)
        self.cmd = ["nvidia-smi", "-i", ident, f"--query-gpu={self.FIELDS}",
                    "--format=csv,noheader,nounits", "-lms", "50"]

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(self.cmd, stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                    power.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": max(mx),
                "power_w_max": max(power), "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ timing helpers

def quantiles(samples):
    s = sorted(samples)
    q = lambda f: s[min(len(s) - 1, int(f * len(s)))]
    return statistics.median(s), q(0.2), q(0.8)


def timed_blocks(fn, steps, warmup, world, device, seconds=2.5, min_blocks=10, max_blocks=40,
                 on_last_block=None):
    """Warm up, then time blocks of exactly ``steps`` calls, each bracketed by a barrier and a
    device synchronisation, max over ranks per block.  Returns per-step milliseconds of every
    block.  ``on_last_block(True/False)`` is called around the last block (event recording)."""
    import torch.distributed as dist

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def block():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync()
        t = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps

    for _ in range(warmup):
        fn()
    first = block()
    nblocks = int(min(max_blocks, max(min_blocks, math.ceil(seconds * 1e3 / max(first * steps, 1e-3)))))
    if world > 1:                                   # the same count on every rank
        t = torch.tensor([nblocks], device=device)
        dist.broadcast(t, src=0)
        nblocks = int(t.item())
    out = [first]
    for i in range(1, nblocks):
        last = i == nblocks - 1
        if last and on_last_block:
            on_last_block(True)
        out.append(block())
        if last and on_last_block:
            on_last_block(False)
    return out


def count_launches(fn):
    """Kernel launches of one call of ``fn``, split into this library's kernels and others
    (cuBLAS, NCCL, torch element-wise).  Counted once outside the timed region from the
    profiler's kernel records; None when the profiler is unavailable."""
    try:
        from torch.profiler import ProfilerActivity, profile
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fn()
            torch.cuda.synchronize()
        ours = other = 0
        for ev in prof.events():
            if getattr(ev, "device_type", None) is None or "cuda" not in str(ev.device_type).lower():
                continue
            name = ev.name or ""
            if name.lower().startswith(("memcpy", "memset")):
                continue
            if "dpk::" in name:
                ours += 1
            else:
                other += 1
        if ours == 0:
            return None
        return ours, other
    except Exception:
        return None


# ------------------------------------------------------------------ CPU legs (oracle)

def cpu_layer_leg(shape, steps, warmup, threads=None):
    """The reference's CPU formulation of the layer (dense products, then mask; the oracle's
    ``dense_then_mask_layer_rows``) on every CPU_SAMPLE_STRIDE-th token row of the sequence,
    K/V of the whole sequence given.  Returns (tokens per step, seconds per step list)."""
    from oracle import dpk_oracle as O

    if threads:
        torch.set_num_threads(threads)
    s = shape
    g = torch.Generator().manual_seed(17)
    H, D, Hq, Hk, T = s.hidden, s.head_dim, s.q_heads, s.kv_heads, s.tokens
    w = {"wq": torch.randn(Hq * D, H, generator=g) * 0.02, "wk": torch.randn(Hk * D, H, generator=g) * 0.02,
         "wv": torch.randn(Hk * D, H, generator=g) * 0.02, "wo": torch.randn(H, Hq * D, generator=g) * 0.02,
         "wg": torch.randn(s.inter, H, generator=g) * 0.02, "wu": torch.randn(s.inter, H, generator=g) * 0.02,
         "wd": torch.randn(H, s.inter, generator=g) * 0.02}
    rows = torch.arange(CPU_SAMPLE_STRIDE - 1, T, CPU_SAMPLE_STRIDE)
    R = rows.numel()
    x = torch.randn(1, T, H, generator=g)
    k = torch.randn(1, T, Hk, D, generator=g)
    v = torch.randn(1, T, Hk, D, generator=g)
    am = O.topk_route_mask(torch.randn(1, R, s.attn_groups, generator=g), s.attn_keep)
    fm = O.topk_route_mask(torch.randn(1, R, s.ffn_groups, generator=g), s.ffn_keep)

    def run():
        t0 = time.perf_counter()
        O.dense_then_mask_layer_rows(x, rows, w, k, v, am, fm, num_q_heads=Hq, num_kv_heads=Hk,
                                     head_dim=D)
        return time.perf_counter() - t0

    for _ in range(warmup):
        run()
    return R, [run() for _ in range(steps)]


def cpu_sample_text(shape, R):
    return (f"{R} of {shape.tokens} token rows per step (every {CPU_SAMPLE_STRIDE}th row, attending "
            "to the keys before it; K/V of the whole sequence given), fp32, dense-then-mask as the "
            "reference's PyTorch path computes it: 1/%d of the layer's work" % CPU_SAMPLE_STRIDE)


def run_reference_arm(args, rank, world):
    """--impl reference: the reference's own CPU implementation of the path (its PyTorch
    backend computes dense products and masks afterwards); here the oracle port, since the
    reference package itself is not present on the GPU box.  Rank 0 alone runs it."""
    if rank != 0:
        return
    from dpk_b200.workloads import LayerShape

    shape = LayerShape(tokens=args.tokens)
    threads = max(1, os.cpu_count() or 1)      # torchrun pins OMP_NUM_THREADS=1 per rank
    R, secs = cpu_layer_leg(shape, args.steps, args.warmup, threads)
    dt = sum(secs) / len(secs)
    val = R / dt
    sample = cpu_sample_text(shape, R) + f", {threads} threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": make_config(shape, world, args),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(),
                         "host_cpus": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------ parity (oracle as checker)

def strict_err(got, want):
    """max|err| / rms(whole expected tensor): the bound as the benchmark states it."""
    from oracle import dpk_oracle as O
    return O.rel_err(got.float().cpu(), want)


def layer_parity(shape, x, fe, host_w, out, am_all, fm_all, nrows=256):
    """Sampled token rows of the layer output against the fp32 CPU oracle run with the routing
    decisions the layer took; the first router's decisions against the oracle's router."""
    from oracle import dpk_oracle as O

    bf = torch.bfloat16
    T = shape.tokens
    rows = torch.randperm(T, generator=torch.Generator().manual_seed(5))[:nrows].sort().values
    xc = x.float().cpu()
    amr, fmr = am_all[:, rows.to(am_all.device)].cpu(), fm_all[:, rows.to(fm_all.device)].cpu()
    kw = dict(num_q_heads=shape.q_heads, num_kv_heads=shape.kv_heads, head_dim=shape.head_dim,
              norm1=fe["n1"].float().cpu(), norm2=fe["n2"].float().cpu(), eps=shape.eps,
              cos=fe["cos"].float().cpu(), sin=fe["sin"].float().cpu())
    want = O.decoder_layer_rows(xc, rows, host_w, amr, fmr, **kw)
    want_h = O.decoder_layer_rows(xc, rows, host_w, amr, fmr, handoff=bf, **kw)
    got = out[:, rows.to(out.device)].float().cpu()
    ra = tuple(t.float().cpu() for t in fe["attn_router"])
    la, ea = O.bottleneck_router(xc[:, rows], *ra, module_dtype=bf)
    clear = (la[..., 0] - la[..., 1]).abs() > 6e-2
    err = O.rel_err(got, want)
    floor = O.rel_err(want_h, want)
    rms = float(want.pow(2).mean().sqrt())
    return {"rows": int(rows.numel()), "max_abs_over_rms": err, "tol": TOL,
            "bf16_handoff_floor": floor, "ok": bool(err <= TOL + floor),
            "criterion": "max|out - fp32 oracle| / rms <= tol + floor, where floor is the same metric for "
                         "the fp32 oracle with every inter-operator tensor rounded to bf16 (what any "
                         "pipeline of bf16 operators pays; the stated tolerance is per operator)",
            "max_abs_over_rms_vs_bf16_handoff_oracle": O.rel_err(got, want_h),
            "rms_err_over_rms": float((got - want).pow(2).mean().sqrt()) / rms, "output_rms": rms,
            "attn_router_decisions_equal_where_clear": bool(torch.equal(amr[clear], ea[clear])),
            "attn_router_clear_fraction": float(clear.float().mean()),
            "kept_fraction": {"attn": float(am_all.float().mean()), "ffn": float(fm_all.float().mean())}}


# ------------------------------------------------------------------ sub-records (N = 1)

def sub_ffn_prefill(dev, steps, peaks):
    """Config 2: Llama-3-8B-shaped dynamic FFN prefill."""
    from dpk_b200 import ops, workloads as W
    from dpk_b200.ffn import RoutedFFN
    from oracle import dpk_oracle as O

    sh = W.FfnShape()
    x, wg, wu, wd, logits = W.ffn_tensors(dev, sh)
    ffn = RoutedFFN(wg, wu, wd, sh.groups, sh.tokens)
    y = torch.empty(sh.tokens, sh.hidden, dtype=torch.bfloat16, device=dev)
    events = {}
    state = {"ev": None}

    def step():
        mask = ops.topk_route_mask(logits, sh.keep)
        ffn(x, mask, out=y, events=state["ev"])

    blocks = timed_blocks(step, steps, 5, 1, dev, seconds=0.6, min_blocks=5, max_blocks=20,
                          on_last_block=lambda on: state.update(ev=events if on else None))
    ms, lo, hi = quantiles(blocks)

    def dense():
        return (torch.nn.functional.silu(x[0] @ wg.T) * (x[0] @ wu.T)) @ wd.T
    dblocks = timed_blocks(dense, steps, 3, 1, dev, seconds=0.3, min_blocks=3, max_blocks=10)
    dms = statistics.median(dblocks)
    k_mn = sum(a.elapsed_time(b) for a, b in events["gemm_mn"]) / len(events["gemm_mn"])
    k_k = sum(a.elapsed_time(b) for a, b in events["gemm_k"]) / len(events["gemm_k"])
    mask = ops.topk_route_mask(logits, sh.keep)
    routing_ok = torch.equal(mask.cpu(), O.topk_route_mask(logits.cpu(), sh.keep))
    rows = torch.randperm(sh.tokens, generator=torch.Generator().manual_seed(1))[:192]
    want = O.ffn_swiglu(x[:, rows].float().cpu(), wg.float().cpu(), wu.float().cpu(), wd.float().cpu(),
                        mask[:, rows].cpu())
    err = strict_err(y[rows][None], want)
    nnz = int(mask.sum())
    f_mn, f_k = 4.0 * sh.hidden * 128 * nnz, 2.0 * sh.hidden * 128 * nnz
    sus, burst = peaks[0], peaks[1]
    return {"workload": sh.name, "ms": ms, "ms_p20_p80": [lo, hi], "tokens_per_s": sh.tokens / (ms * 1e-3),
            "dense_ms": dms, "speedup_vs_dense": dms / ms,
            "gemm_mn_ms": k_mn, "gemm_k_ms": k_k,
            "roofline": {"kernel": "gemm_mn_pair_kernel", "bound": "tensor", "achieved": f_mn / (k_mn * 1e-3) / 1e12,
                         "peak": burst, "unit": "TFLOP/s", "frac": f_mn / (k_mn * 1e-3) / 1e12 / burst,
                         "peak_source": "measured burst bf16 (sub-millisecond kernel)",
                         "frac_of_sustained": f_mn / (k_mn * 1e-3) / 1e12 / sus},
            "gemm_k_algorithmic_tflops": f_k / (k_k * 1e-3) / 1e12,
            "parity": {"rows": 192, "max_abs_over_rms": err, "tol": TOL, "ok": bool(err <= TOL),
                       "routing_bit_exact": bool(routing_ok)}}


def sub_attention_prefill(dev, steps, peaks):
    """Config 3: head-group-routed causal prefill attention."""
    from dpk_b200 import ops, workloads as W
    from oracle import dpk_oracle as O

    sh = W.PrefillShape()
    q, k, v, logits = W.prefill_tensors(dev, sh)
    mask = ops.topk_route_mask(logits, sh.keep)
    out = torch.zeros_like(q)

    def step():
        ops.attention_prefill(q, k, v, mask, O=out)
    blocks = timed_blocks(step, steps, 5, 1, dev, seconds=0.4, min_blocks=5, max_blocks=20)
    ms, lo, hi = quantiles(blocks)
    sdpa = torch.nn.functional.scaled_dot_product_attention
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    dblocks = timed_blocks(lambda: sdpa(qt, kt, vt, is_causal=True, enable_gqa=True), steps, 3, 1, dev,
                           seconds=0.3, min_blocks=3, max_blocks=10)
    dms = statistics.median(dblocks)
    # exact algorithmic flops for this mask: 4*D per (active query row of a head, visible key)
    pos = torch.arange(1, sh.tokens + 1, device=dev, dtype=torch.float64)
    pairs = float((mask[0].to(torch.float64) * pos[:, None]).sum()) * (sh.q_heads // sh.groups)
    flops = 4.0 * sh.head_dim * pairs
    ach = flops / (ms * 1e-3) / 1e12
    rows = torch.randperm(sh.tokens, generator=torch.Generator().manual_seed(2))[:256].sort().values
    rd = rows.to(dev)
    want = O.attention(q[:, rd].float().cpu(), k.float().cpu(), v.float().cpu(), mask[:, rd].cpu(),
                       is_causal=True, q_positions=rows)
    got = out[:, rd].float().cpu()
    err, err_rows = O.rel_err(got, want), O.rel_err_rows(got, want)
    routing_ok = torch.equal(mask.cpu(), O.topk_route_mask(logits.cpu(), sh.keep))
    return {"workload": sh.name, "ms": ms, "ms_p20_p80": [lo, hi], "tokens_per_s": sh.tokens / (ms * 1e-3),
            "dense_sdpa_ms": dms, "speedup_vs_dense": dms / ms, "algorithmic_tflop": flops / 1e12,
            "roofline": {"kernel": "attn_prefill_tc_kernel", "bound": "tensor", "achieved": ach,
                         "peak": peaks[1], "unit": "TFLOP/s", "frac": ach / peaks[1],
                         "peak_source": "measured burst bf16 (sub-millisecond kernel)",
                         "frac_of_sustained": ach / peaks[0]},
            "parity": {"rows": 256, "max_abs_over_rms": err, "max_over_rows_of_abs_over_row_rms": err_rows,
                       "tol": TOL, "ok": bool(err_rows <= TOL), "routing_bit_exact": bool(routing_ok),
                       "note": "the tolerance is met per output row; the global-RMS form is printed beside it"}}


def sub_decode(dev, steps, peaks):
    """Config 4: one decode step -- routed attention over the KV cache and the decode FFN."""
    from dpk_b200 import ops, workloads as W
    from dpk_b200.ffn import RoutedFFN
    from oracle import dpk_oracle as O

    sh = W.DecodeShape()
    q, k, v, logits = W.decode_tensors(dev, sh)
    amask = ops.topk_route_mask(logits, sh.attn_keep)
    f = sh.ffn
    x, wg, wu, wd, flogits = W.ffn_tensors(dev, f)
    x = x.view(f.tokens, 1, f.hidden)
    fmask = ops.topk_route_mask(flogits.view(f.tokens, 1, f.groups), f.keep)
    ffn = RoutedFFN(wg, wu, wd, f.groups, f.tokens)
    o = torch.empty_like(q)
    y = torch.empty(f.tokens, f.hidden, dtype=torch.bfloat16, device=dev)
    a_blocks = timed_blocks(lambda: ops.attention_decode(q, k, v, amask, O=o), steps, 5, 1, dev,
                            seconds=0.4, min_blocks=5, max_blocks=20)
    f_blocks = timed_blocks(lambda: ffn(x, fmask, out=y), steps, 5, 1, dev, seconds=0.2, min_blocks=5,
                            max_blocks=20)
    a_ms, f_ms = statistics.median(a_blocks), statistics.median(f_blocks)
    # the same two calls as ONE CUDA graph, replayed: how the reference times its kernels
    # (gemm_mn/jit.py:619-631), and what a decode loop would launch per layer
    graph_ms = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            ops.attention_decode(q, k, v, amask, O=o)
            ffn(x, fmask, out=y)
        graph_ms = statistics.median(timed_blocks(graph.replay, steps, 5, 1, dev, seconds=0.4, min_blocks=5,
                                                  max_blocks=20))
    except Exception as exc:       # capture is an extra, not the measurement
        print(f"bench: CUDA graph capture of the decode step failed: {exc}", file=sys.stderr)
    sdpa = torch.nn.functional.scaled_dot_product_attention
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    d_ms = statistics.median(timed_blocks(lambda: sdpa(qt, kt, vt, enable_gqa=True), steps, 3, 1, dev,
                                          seconds=0.2, min_blocks=3, max_blocks=8))
    # a KV head is read when any of the head groups that use it is active
    if sh.attn_groups >= sh.kv_heads:
        n_active = int(amask.view(sh.batch, sh.kv_heads, -1).any(-1).sum())
    else:
        n_active = int(amask.sum()) * (sh.kv_heads // sh.attn_groups)
    a_bytes = 2.0 * sh.kv_len * sh.head_dim * 2 * n_active
    f_bytes = 3.0 * f.hidden * f.inter * 2
    hbm = peaks[2]
    a_gbs, f_gbs = a_bytes / (a_ms * 1e-3) / 1e9, f_bytes / (f_ms * 1e-3) / 1e9
    # parity: 8 sampled sequences, all heads; the FFN on all 64 tokens
    seqs = torch.randperm(sh.batch, generator=torch.Generator().manual_seed(3))[:8].sort().values
    sd = seqs.to(dev)
    want = O.attention_decode(q[sd].float().cpu(), k[sd].float().cpu(), v[sd].float().cpu(), amask[sd].cpu())
    got = o[sd].float().cpu()
    err, err_rows = O.rel_err(got, want), O.rel_err_rows(got, want)
    wantf = O.ffn_swiglu(x.float().cpu(), wg.float().cpu(), wu.float().cpu(), wd.float().cpu(), fmask.cpu())
    errf = strict_err(y.view(f.tokens, 1, f.hidden), wantf)
    return {"workload": sh.name, "tpot_us": (a_ms + f_ms) * 1e3, "attention_us": a_ms * 1e3, "ffn_us": f_ms * 1e3,
            "tpot_cuda_graph_us": graph_ms * 1e3 if graph_ms else None,
            "dense_sdpa_us": d_ms * 1e3, "attention_speedup_vs_dense": d_ms / a_ms,
            "floor_us": (a_bytes + f_bytes) / (hbm * 1e9) * 1e6,
            "roofline": {"kernel": "attn_decode_kernel", "bound": "hbm", "achieved": a_gbs, "peak": hbm,
                         "unit": "GB/s", "frac": a_gbs / hbm, "peak_source": "measured copy bandwidth",
                         "algorithmic_bytes_per_launch": a_bytes},
            "ffn_hbm_gbs": f_gbs, "ffn_frac": f_gbs / hbm,
            "l2": "K/V 8 GiB and FFN weights 352 MB per step: larger than L2",
            "parity": {"sequences": 8, "attention_max_abs_over_rms": err,
                       "attention_max_over_rows_of_abs_over_row_rms": err_rows,
                       "ffn_max_abs_over_rms": errf, "tol": TOL,
                       "ok": bool(err_rows <= TOL and errf <= TOL)}}


# ------------------------------------------------------------------ main arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=16384,
                    help="sequence length (default: the benchmark's 16384; smaller values are for "
                         "profiler captures only and show in config.workload)")
    ap.add_argument("--sum", choices=["fused", "nccl"], default="fused",
                    help="N > 1: how the ranks' partial outputs are added: 'fused' = the projection "
                         "stores its partial token windows into the owning rank's memory and a "
                         "reduce+gather kernel finishes the sum; 'nccl' = NCCL all-reduce")
    ap.add_argument("--halves", type=int, default=2, choices=[1, 2],
                    help="--sum fused: 2 = project the tokens in two halves and gather the first half "
                         "under the second half's projection")
    ap.add_argument("--barrier", choices=["nccl", "flags"], default="nccl",
                    help="--sum fused: what separates the two kernels of a sum on the stream: a "
                         "one-element NCCL all-reduce, or dpk_peer_barrier (flags in peer memory)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the sub-records of configs 2-4")
    ap.add_argument("--skip-e2e", action="store_true", help="profiler captures only")
    ap.add_argument("--skip-dense", action="store_true", help="profiler captures only")
    ap.add_argument("--mn-gather", type=int, default=-1, choices=[-1, 0, 1],
                    help="measurements only: token rows of the output-width GEMM by cp.async (0) or TMA "
                         "tile::gather4 (1); -1 = the library's default")
    ap.add_argument("--attn-heads", type=int, default=0, choices=[0, 1, 2],
                    help="measurements only: 2 = the prefill attention kernel with two query heads per CTA")
    ap.add_argument("--one-block", action="store_true",
                    help="profiler captures only: time a single block of --steps steps")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    from dpk_b200 import build as _build
    if rank == 0:
        _build.build()
    if world > 1:
        dist.barrier()
    from dpk_b200 import ops, workloads as W
    if args.mn_gather >= 0 or args.attn_heads:
        from dpk_b200 import _native
        if args.mn_gather >= 0:
            _native.check(_native.load().dpk_set_gemm_mn_gather(args.mn_gather))
        _native.check(_native.load().dpk_set_attn_prefill_heads(args.attn_heads))

    # ---- sub-records of the other configurations (single GPU), before the long loops of the
    # layer heat the GPU into its power cap: these are sub-millisecond kernels, timed as a burst
    peaks = measured_peaks()
    configs = None
    if world == 1 and not args.no_configs and args.tokens == 16384:
        configs = {"c2": sub_ffn_prefill(device, args.steps, peaks)}
        torch.cuda.empty_cache()
        configs["c3"] = sub_attention_prefill(device, args.steps, peaks)
        torch.cuda.empty_cache()
        configs["c4"] = sub_decode(device, args.steps, peaks)
        torch.cuda.empty_cache()
        status = ops.device_status()
        if status:
            raise SystemExit(f"sub-records: a kernel reported status {status}")

    shape = W.LayerShape(tokens=args.tokens)
    T, H = shape.tokens, shape.hidden
    if shape.attn_groups % world or shape.ffn_groups % world or T % world:
        raise SystemExit(f"the layer does not split over {world} ranks")
    want_parity = not args.no_parity
    layer, fe, host_w = W.build_layer(device, shape, world, rank,
                                      keep_host_fp32=want_parity and rank == 0)
    x = W.layer_input(device, shape)
    cos, sin = fe["cos"], fe["sin"]

    def all_ranks_ok(flag: bool) -> bool:
        if world == 1:
            return flag
        t = torch.tensor([0 if flag else 1], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return int(t.item()) == 0

    def check_status(where: str):
        """Every rank leaves together when any rank's kernels reported a problem."""
        status = ops.device_status()
        t = torch.tensor([status], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if int(t.item()) != 0:
            if world > 1:
                dist.destroy_process_group()
            raise SystemExit(f"{where}: a kernel reported status {int(t.item())} (this rank: {status})")

    # ---- N > 1: the sums with NCCL first (cross-check), then fused ---------------------------
    # The check runs the operators with GIVEN routing masks (top-k of seeded logits): with the
    # layer's own routers a last-bit difference in the summed hidden state flips decisions that
    # sit on the boundary, which would be a routing difference, not a difference of the sums.
    sum_check = None
    fused = False
    if world > 1:
        (ga0, ga1), (gf0, gf1) = shape.shard(world, rank)
        gm = torch.Generator(device=device).manual_seed(29)
        am_chk = ops.topk_route_mask(torch.randn(1, T, shape.attn_groups, generator=gm, device=device),
                                     shape.attn_keep)[..., ga0:ga1]
        fm_chk = ops.topk_route_mask(torch.randn(1, T, shape.ffn_groups, generator=gm, device=device),
                                     shape.ffn_keep)[..., gf0:gf1]
        out_nccl = layer(x, am_chk, fm_chk).clone()
        if args.sum == "fused":
            try:
                layer.fuse_sums(T)
                layer.sum_o.halves = layer.ffn.row_parallel.halves = args.halves
                layer.sum_o.barrier_mode = layer.ffn.row_parallel.barrier_mode = args.barrier
                fused = True
            except RuntimeError as exc:       # the same exception on every rank (see connect)
                if rank == 0:
                    print(f"bench: {exc}; summing the partial outputs with NCCL instead", file=sys.stderr)
        if fused:
            out_fused = layer(x, am_chk, fm_chk)
            a, b = out_fused.float(), out_nccl.float()
            rms_b = b.pow(2).mean().sqrt()
            rel = torch.stack([(a - b).abs().max() / rms_b, (a - b).pow(2).mean().sqrt() / rms_b])
            digest = out_fused.view(torch.int16).to(torch.int64).sum().reshape(1)
            digests = [torch.empty_like(digest) for _ in range(world)]
            dist.all_gather(digests, digest)
            same = all(int(d.item()) == int(digests[0].item()) for d in digests)
            dist.all_reduce(rel, op=dist.ReduceOp.MAX)
            rel_max, rel_rms = float(rel[0].item()), float(rel[1].item())
            # NCCL adds bf16 partial sums in bf16 (every rank's partial is rounded, and so is every
            # hop of the reduction), the fused sum adds in fp32 and rounds once: single entries
            # differ by a few bf16 ulps of the largest values (the maximum below), but the RMS of
            # the difference stays at rounding level (measured 6e-3 at 4 ranks).  One misplaced
            # 128-token window out of 16384 tokens would put it near 1e-1, so the RMS bound is the
            # check; the precise check of the fused output is the "parity" record against the oracle.
            bound = 2e-2
            sum_check = {"fused_vs_nccl_rms_diff_over_rms": rel_rms, "bound": bound,
                         "fused_vs_nccl_max_abs_over_rms": rel_max,
                         "identical_output_on_every_rank": bool(same),
                         "ok": bool(rel_rms <= bound and same),
                         "how": "the layer's operators with given top-k masks, NCCL all-reduces (bf16 arithmetic) "
                                "against the fused row-parallel sums (fp32, one rounding)"}
            del out_fused
        del out_nccl, am_chk, fm_chk
        check_status("cross-check of the sums")

    def step():
        return layer.forward_full(x, cos, sin)

    # ---- device-resident timing -----------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    layer.ffn_events = None
    events = {}

    phase_timers = {}

    def last_block(on):
        # CUDA events around the phases and the two FFN GEMM kernels, last timed block only
        layer.timers = phase_timers if on else None
        layer.ffn_events = events if on else None

    blocks = timed_blocks(step, args.steps, args.warmup, world, device,
                          seconds=0.0 if args.one_block else 2.5,
                          min_blocks=1 if args.one_block else 10, on_last_block=last_block)
    clocks_device = sampler.stop() if rank == 0 else None
    check_status("device-resident loop")
    ms_step, ms_lo, ms_hi = quantiles(blocks)

    def mean_ms(pairs):
        return sum(a.elapsed_time(b) for a, b in pairs) / len(pairs)

    k_mn = mean_ms(events["gemm_mn"]) if events.get("gemm_mn") else None
    k_k = mean_ms(events["gemm_k"]) if events.get("gemm_k") else None
    phases = {}
    tm = phase_timers
    names = ["start", "route1", "qkv", "attn", "oproj", "route2", "ffn"]
    if all(n in tm for n in names):
        for a, b in zip(names[:-1], names[1:]):
            phases[b + "_ms"] = sum(e0.elapsed_time(e1) for e0, e1 in zip(tm[a], tm[b])) / len(tm[a])

    # ---- masks, launches, parity (outside the timed region) ---------------------------------
    out, am_all, fm_all = layer.forward_full(x, cos, sin, return_masks="full")
    (ga0, ga1), (gf0, gf1) = shape.shard(world, rank)
    nnz_f_local = int(fm_all[..., gf0:gf1].sum())
    nnz_f, nnz_a = int(fm_all.sum()), int(am_all.sum())
    pos = torch.arange(1, T + 1, device=device, dtype=torch.float64)
    attn_pairs = float((am_all[0].to(torch.float64) * pos[:, None]).sum()) * (shape.q_heads // shape.attn_groups)
    launches = count_launches(step)
    parity = None
    if want_parity and rank == 0:
        parity = layer_parity(shape, x, fe, host_w, out, am_all, fm_all)
        host_w = None
    if sum_check is not None and parity is not None:
        parity["sums"] = sum_check
    check_status("parity pass")

    # ---- end to end with host buffers: every rank moves its own rows over its own PCIe link --
    e2e = None
    rows_r = T // world
    r0 = rank * rows_r
    if not args.skip_e2e:
        x_host = W.layer_input(device, shape, host=True)[0, r0:r0 + rows_r]
        xh = [x_host.pin_memory(), x_host.clone().pin_memory()]
        yh = [torch.empty(rows_r, H, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        xs = [torch.empty(rows_r, H, dtype=torch.bfloat16, device=device) for _ in range(2)]
        xd = [torch.empty(1, T, H, dtype=torch.bfloat16, device=device) for _ in range(2)]
        yd = [torch.empty(rows_r, H, dtype=torch.bfloat16, device=device) for _ in range(2)]
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        s_cmp = torch.cuda.current_stream()

        def e2e_loop(n):
            ev_in, ev_cmp, ev_out = [None, None], [None, None], [None, None]
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if ev_cmp[b] is not None:
                        s_in.wait_event(ev_cmp[b])            # input buffer b is free again
                    (xs[b] if world > 1 else xd[b][0]).copy_(xh[b], non_blocking=True)
                    ev_in[b] = torch.cuda.Event()
                    ev_in[b].record(s_in)
                s_cmp.wait_event(ev_in[b])
                if world > 1:
                    # the row blocks reach the other ranks over NVLink
                    dist.all_gather_into_tensor(xd[b].view(T, H), xs[b])
                if ev_out[b] is not None:
                    s_cmp.wait_event(ev_out[b])               # output buffer b has been read back
                res = layer.forward_full(xd[b], cos, sin)
                yd[b].copy_(res[0, r0:r0 + rows_r])           # every rank holds all rows; it returns its block
                ev_cmp[b] = torch.cuda.Event()
                ev_cmp[b].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[b])
                    yh[b].copy_(yd[b], non_blocking=True)
                    ev_out[b] = torch.cuda.Event()
                    ev_out[b].record(s_out)

        e2e_loop(args.warmup)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        if rank == 0:
            sampler = ClockSampler(local_rank)
            sampler.start()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        g0.record(s_in)
        e2e_loop(args.steps)
        s_out.synchronize()
        g1.record(s_out)
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3
        if world > 1:
            dist.barrier()
        e2e_ms = max(g0.elapsed_time(g1), 0.0)
        if not (0.5 * wall_ms <= e2e_ms <= 1.5 * wall_ms):
            e2e_ms = wall_ms                     # events on two streams disagree with the host clock
        t = torch.tensor([e2e_ms], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms_step = float(t.item()) / args.steps
        clocks_e2e = sampler.stop() if rank == 0 else None
        check_status("end-to-end loop")
        e2e = {"value": T / (e2e_ms_step * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms_step,
               "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": T * H * 2,
               "how": ("pinned host x -> device, the layer, output -> pinned host, double buffered over "
                       "3 streams" if world == 1 else
                       f"every rank copies its {rows_r} rows of x from pinned host memory over its own PCIe "
                       "link, an NVLink all-gather completes x on every rank, the layer runs, every rank "
                       "copies its rows of the output back; double buffered over 3 streams"),
               "clocks": clocks_e2e}
        del xh, yh, xs, xd, yd

    # ---- the same layer without routing (cuBLAS, SDPA, NCCL all-reduce), same sharding -----
    dense = None
    if not args.skip_dense:
        wo = layer.wo
        wg, wu, wd = layer.ffn.wg, layer.ffn.wu, layer.ffn.wd
        n1, n2 = fe["n1"], fe["n2"]
        D, hq_l, hk_l = shape.head_dim, layer.Hq, layer.Hk
        sdpa = torch.nn.functional.scaled_dot_product_attention

        wqkv = layer.wqkv                       # [Wq; Wk; Wv] stacked: one library GEMM
        qd, kd = hq_l * D, hk_l * D

        def dense_step():
            # the glue is as lean as the routed layer's: one stacked q/k/v GEMM, this library's
            # rotary kernel in place on the slices, residual adds inside the GEMMs (addmm) where
            # no all-reduce comes between
            xf = x[0]
            xn = torch.nn.functional.rms_norm(xf, (H,), n1, shape.eps)
            qkv = (xn @ wqkv.T).view(1, T, qd + 2 * kd)
            q = qkv[..., :qd].view(1, T, hq_l, D)
            k = qkv[..., qd:qd + kd].view(1, T, hk_l, D)
            v = qkv[..., qd + kd:].view(1, T, hk_l, D)
            ops.rope_append(q, k, None, cos, sin)
            a = sdpa(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                     enable_gqa=True).transpose(1, 2).reshape(T, hq_l * D)
            if world > 1:
                o = a @ wo.T
                dist.all_reduce(o)
                x1 = xf + o
            else:
                x1 = torch.addmm(xf, a, wo.T)
            x1n = torch.nn.functional.rms_norm(x1, (H,), n2, shape.eps)
            hmid = torch.nn.functional.silu(x1n @ wg.T) * (x1n @ wu.T)
            if world > 1:
                yy = hmid @ wd.T
                dist.all_reduce(yy)
                return x1 + yy
            return torch.addmm(x1, hmid, wd.T)

        dblocks = timed_blocks(dense_step, args.steps, 3, world, device, seconds=1.0, min_blocks=3,
                               max_blocks=10)
        dms = statistics.median(dblocks)
        dense = {"value": T / (dms * 1e-3), "unit": UNIT, "ms_per_step": dms,
                 "what": "the same layer with every group kept: rms_norm, one stacked q/k/v GEMM and the other "
                         "projections by cuBLAS bf16 (residual adds inside addmm), this library's rotary "
                         "kernel, SDPA causal, silu*mul" +
                         (", NCCL all-reduce of both partial sums" if world > 1 else "")}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    sus, burst, hbm, peak_src = peaks
    # algorithmic flops of the whole layer (all ranks), from the decisions of this run
    hpg_ch = shape.q_heads // shape.attn_groups * shape.head_dim
    flops = (6.0 * H * 128 * nnz_f                                   # FFN
             + 4.0 * shape.head_dim * attn_pairs                     # attention
             + 2.0 * 2.0 * H * hpg_ch * nnz_a                        # Q and O projections
             + 2.0 * 2.0 * H * shape.kv_heads * shape.head_dim * T)  # dense K, V projections
    value = T / (ms_step * 1e-3)
    roof = None
    if k_mn:
        flops_mn = 4.0 * H * 128 * nnz_f_local
        ach = flops_mn / (k_mn * 1e-3) / 1e12
        roof = {"kernel": "gemm_mn_pair_kernel (fused gate/up + SwiGLU, CTA pairs)", "bound": "tensor",
                "achieved": ach, "peak": sus, "unit": "TFLOP/s", "frac": ach / sus,
                "peak_source": f"{peak_src} sustained bf16: the kernel is timed inside a seconds-long loop "
                               "of layer steps (see clocks)",
                "frac_of_burst_peak": ach / burst, "traffic": recorded_traffic(shape, world),
                "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch of this shape "
                                  "under ncu, read from profiles/gemm_mn_pair_config5_counters.md (not "
                                  "measured by this run; null for other shapes)",
                "algorithmic_flops_per_launch": flops_mn, "launch_ms": k_mn}
    roof_down = None
    if k_k and world == 1:
        # the other large kernel: the down projection (reduction-width routed).  Rows of tokens that
        # do not use a group still occupy MMA rows of their window's tile, so at a keep fraction f
        # it executes 1/f times its algorithmic flops (every window visits every group here).
        flops_k = 2.0 * H * 128 * nnz_f_local
        executed = 2.0 * H * (shape.ffn_groups * 128.0) * T
        roof_down = {"kernel": "gemm_k_pair_kernel (down projection + skip connection, CTA pairs)",
                     "bound": "tensor", "achieved": flops_k / (k_k * 1e-3) / 1e12, "peak": sus,
                     "unit": "TFLOP/s", "frac": flops_k / (k_k * 1e-3) / 1e12 / sus,
                     "executed_tflops": executed / (k_k * 1e-3) / 1e12,
                     "executed_frac": executed / (k_k * 1e-3) / 1e12 / sus,
                     "algorithmic_flops_per_launch": flops_k, "launch_ms": k_k}
    cpu = None
    if not args.no_cpu_baseline and world == 1:
        R, secs = cpu_layer_leg(shape, 3, 1)
        dt = statistics.median(secs)
        cpu = {"value": R / dt, "unit": UNIT, "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(),
               "kind": "port", "sample": cpu_sample_text(shape, R) + f"; {dt:.2f} s per step"}
    ours_l, other_l = launches if launches else (None, None)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": make_config(shape, world, args),
        "timing": {"blocks": len(blocks), "steps_per_block": args.steps, "ms_per_step_p20_p80": [ms_lo, ms_hi],
                   "how": "median over blocks of (max over ranks of a block's device time) / steps"},
        "sums": ("fused row-parallel sums, tokens in %d part(s), %s barriers" % (args.halves, args.barrier)) if fused else
                ("NCCL all-reduce" if world > 1 else None),
        "algorithmic_tflop_per_step": flops / 1e12,
        "layer_roofline": {"achieved": flops / (ms_step * 1e-3) / 1e12, "peak": sus * world, "unit": "TFLOP/s",
                           "frac": flops / (ms_step * 1e-3) / 1e12 / (sus * world),
                           "peak_source": f"{peak_src} sustained bf16 x {world} GPU(s)"},
        "roofline": roof,
        "roofline_down_projection": roof_down,
        "kernels": {"gemm_mn_ms": k_mn, "gemm_k_ms": k_k,
                    "gemm_k_ms_covers": ("down projection + barriers + reduce/gather" if fused else "down projection"),
                    "phases_ms": phases},
        "clocks": clocks_device,
        "e2e": e2e,
        "parity": parity,
        "gpu_launches": (ours_l * args.steps) if ours_l else None,
        "launches_per_step": {"this_library": ours_l, "other (torch element-wise ops on masks and residuals, NCCL)": other_l},
    }
    if dense is not None:
        line["dense"] = dense
        line["speedup_vs_dense"] = value / dense["value"]
    if configs is not None:
        line["configs"] = configs
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
