#!/usr/bin/env python
"""Benchmark of the routed dynamic-width FFN path (Llama-3-8B-shaped FFN prefill, 8192 tokens).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): Llama-3-8B-shaped dynamic FFN prefill -- hidden 4096, intermediate
14336 as 112 groups of 128 channels, 8192 tokens, per-token top-56 groups from seeded
N(0,1) router logits, bf16 activations N(0,1), weights N(0,0.02); synthetic data.
One step = top-k router mask + routing layout + packed bits + fused gate/up GEMM
(SwiGLU epilogue) + reduction-width down GEMM.  With N > 1 the same layer is
tensor-parallel by channel groups (rank r owns NG/N groups: rows of the gate/up
weights, columns of the down weight) with one NCCL all-reduce of the partial outputs;
total work is fixed (strong scaling).

Prints ONE JSON line on rank 0.  Keys beyond the common contract:
  roofline      dominant kernel (fused gate/up GEMM) against the measured bf16 peak
  kernels       per-kernel mean launch time inside the timed region (CUDA events)
  dense         the dense cuBLAS bf16 equivalent (3 matmuls + silu*mul), same run
  cpu_baseline  the reference's CPU formulation (dense, then mask) on the host cores
  e2e           the same metric with host buffers: pinned H2D of x and the router
                logits and D2H of y inside the timed region, double buffered
"""

from __future__ import annotations

import argparse
import json
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

M_TOK, HID, INTER, NGROUPS, KEEP = 8192, 4096, 14336, 112, 56
SEED = 17
METRIC = "prefill_tokens_per_s_dynamic_ffn_layer"
UNIT = "tokens/s"
WORKLOAD = "llama3-8b-ffn-prefill: H=4096 I=14336 NG=112x128 tokens=8192 top-56 (50% keep)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("bf16_tflops_sustained", 1425.8), d.get("hbm_gbs", 6449.1), "measured"
    return 1400.0, 6650.0, "fallback"


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
                    "--format=csv,noheader,nounits", "-lms", "100"]

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(self.cmd, stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
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
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "samples": len(sm),
                "reasons": sorted(reasons)}


# ------------------------------------------------------------------ inputs

def make_inputs(device, rank_groups=None):
    """Seeded synthetic tensors of the benchmark's shapes and distributions.  Weights are
    drawn on the device (336 MiB of random numbers); x and the router logits on the
    host so that the end-to-end leg starts from host memory."""
    g = torch.Generator().manual_seed(SEED)
    x_host = torch.randn(M_TOK, HID, generator=g).to(torch.bfloat16)
    logits_host = torch.randn(M_TOK, NGROUPS, generator=g)
    dg = torch.Generator(device=device).manual_seed(SEED)
    wg = (torch.randn(INTER, HID, generator=dg, device=device) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(INTER, HID, generator=dg, device=device) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(HID, INTER, generator=dg, device=device) * 0.02).to(torch.bfloat16)
    if rank_groups is not None:
        g0, g1 = rank_groups
        c0, c1 = g0 * 128, g1 * 128
        wg, wu, wd = wg[c0:c1].contiguous(), wu[c0:c1].contiguous(), wd[:, c0:c1].contiguous()
    return x_host, logits_host, wg, wu, wd


# ------------------------------------------------------------------ CPU baseline

def cpu_baseline(seconds: float = 12.0):
    """Times the reference CPU formulation (dense GEMMs, then mask; the oracle's
    ``dense_then_mask_ffn``) on a bounded token sample of the same layer."""
    from oracle import dpk_oracle as O

    g = torch.Generator().manual_seed(SEED)
    wg = torch.randn(INTER, HID, generator=g) * 0.02
    wu = torch.randn(INTER, HID, generator=g) * 0.02
    wd = torch.randn(HID, INTER, generator=g) * 0.02

    def run(tokens):
        x = torch.randn(1, tokens, HID, generator=g)
        mask = O.topk_route_mask(torch.randn(1, tokens, NGROUPS, generator=g), KEEP)
        t0 = time.perf_counter()
        O.dense_then_mask_ffn(x, wg, wu, wd, mask)
        return time.perf_counter() - t0

    run(64)                                  # warm the thread pool
    t = run(256)
    tokens = int(min(8192, max(256, 256 * seconds / max(t, 1e-3))))
    tokens = (tokens // 128) * 128
    t = run(tokens)
    return {"value": tokens / t, "unit": UNIT, "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": "port",
            "sample": f"{tokens} of {M_TOK} tokens of the same layer, fp32, dense-then-mask "
                      f"as the reference's PyTorch path computes it; {t:.2f} s"}


def run_reference_arm(args, rank, world):
    """--impl reference: the reference's own CPU implementation of the path (its PyTorch
    backend computes dense GEMMs and masks afterwards); here the oracle port, since the
    reference package itself is not present on the GPU box."""
    if rank != 0:
        return
    from oracle import dpk_oracle as O

    # torchrun pins OMP_NUM_THREADS=1 per rank; this arm runs on rank 0 alone and may use
    # every host core
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    g = torch.Generator().manual_seed(SEED)
    wg = torch.randn(INTER, HID, generator=g) * 0.02
    wu = torch.randn(INTER, HID, generator=g) * 0.02
    wd = torch.randn(HID, INTER, generator=g) * 0.02
    tokens = 512
    x = torch.randn(1, tokens, HID, generator=g)
    mask = O.topk_route_mask(torch.randn(1, tokens, NGROUPS, generator=g), KEEP)
    for _ in range(args.warmup):
        O.dense_then_mask_ffn(x, wg, wu, wd, mask)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.dense_then_mask_ffn(x, wg, wu, wd, mask)
    dt = (time.perf_counter() - t0) / args.steps
    val = tokens / dt
    sample = f"{tokens} of {M_TOK} tokens per step, fp32, all host threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 * (M_TOK / tokens),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(),
                         "host_cpus": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------ main arm

def main():
    global M_TOK, WORKLOAD
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tokens", type=int, default=8192,
                    help="token count (default: the benchmark's 8192; smaller values are for "
                         "profiler captures only and are named in config.workload)")
    ap.add_argument("--skip-e2e", action="store_true", help="profiler captures only")
    ap.add_argument("--skip-dense", action="store_true", help="profiler captures only")
    ap.add_argument("--sum", choices=["fused", "nccl"], default="fused",
                    help="N > 1: how the ranks' partial outputs are added: 'fused' = the down "
                         "projection stores its partial windows into the owning rank's memory and a "
                         "reduce+gather kernel finishes the sum; 'nccl' = NCCL all-reduce")
    ap.add_argument("--halves", type=int, default=2, choices=[1, 2],
                    help="--sum fused: 2 = project the tokens in two halves and gather the first half "
                         "under the second half's projection")
    ap.add_argument("--ar-chunks", type=int, default=0,
                    help="N > 1: token chunks of the down projection whose all-reduces overlap "
                         "the next chunk's compute (0 = automatic: 4 chunks on 2 GPUs, where the "
                         "16 MiB pieces still run at bandwidth; 1 beyond, where an 8-rank "
                         "all-reduce of a small piece is latency bound and chunking measured slower)")
    ap.add_argument("--sm-margin", type=int, default=-1,
                    help="N > 1: SMs the persistent GEMM kernels leave to the collective "
                         "(-1 = automatic: 8 when chunking, else 0)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.tokens != M_TOK:
        M_TOK = args.tokens
        WORKLOAD = WORKLOAD.replace("tokens=8192", f"tokens={M_TOK} (reduced, not the benchmark size)")

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
    if NGROUPS % world:
        raise SystemExit(f"{NGROUPS} groups do not split over {world} ranks")

    from dpk_b200 import build as _build
    if rank == 0:
        _build.build()
    if world > 1:
        dist.barrier()
    from dpk_b200 import ops
    from dpk_b200.ffn import RoutedFFN

    gpr = NGROUPS // world
    groups = (rank * gpr, (rank + 1) * gpr)
    x_host, logits_host, wg, wu, wd = make_inputs(device, groups if world > 1 else None)
    ffn = RoutedFFN(wg, wu, wd, gpr, M_TOK)
    x = x_host.to(device)
    logits = logits_host.to(device)
    y = torch.empty(M_TOK, HID, dtype=torch.bfloat16, device=device)

    fused = world > 1 and args.sum == "fused"
    if fused:
        from dpk_b200.peer import RowParallelSum
        try:
            ffn.row_parallel = RowParallelSum.connect(M_TOK, HID, torch.bfloat16, device)
            ffn.row_parallel.halves = args.halves
            args.ar_chunks, args.sm_margin = 1, 0
        except RuntimeError as exc:       # the same exception on every rank (see connect)
            if rank == 0:
                print(f"bench: {exc}; summing the partial outputs with NCCL instead", file=sys.stderr)
            fused = False
    if args.ar_chunks <= 0:
        args.ar_chunks = 4 if world == 2 else 1
    chunks = args.ar_chunks if world > 1 else 1
    if args.sm_margin < 0:
        args.sm_margin = 8 if chunks > 1 else 0
    if world > 1:
        from dpk_b200 import _native
        _native.check(_native.load().dpk_set_sm_margin(args.sm_margin))

    def step(events=None, x_in=x, logits_in=logits, y_out=y):
        mask = ops.topk_route_mask(logits_in, KEEP)              # [M, NG] bool, replicated
        if world == 1:
            ffn(x_in, mask, out=y_out, events=events)
            return y_out
        if fused:
            return ffn(x_in, mask[:, groups[0]:groups[1]], events=events)    # shared output buffer
        works = []
        ffn(x_in, mask[:, groups[0]:groups[1]], out=y_out, events=events, row_chunks=chunks,
            chunk_done=lambda rows: works.append(dist.all_reduce(rows, async_op=True)))
        for wk in works:
            wk.wait()
        return y_out

    launches_per_step = 1 + ffn.launches_per_call + ((2 * args.halves - 1) if fused else chunks - 1)

    # ---- device-resident timing -----------------------------------------------------
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    events = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step(events)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    status = ops.device_status()
    if status != 0:
        raise SystemExit(f"a kernel reported status {status}")

    def mean_ms(pairs):
        return sum(a.elapsed_time(b) for a, b in pairs) / len(pairs)

    k_mn = mean_ms(events["gemm_mn"])
    k_k = mean_ms(events["gemm_k"])

    # ---- end to end with host buffers (pinned H2D of x + logits, D2H of y) ---------
    if args.skip_e2e:
        e2e_ms_step = None
    xh = [x_host.pin_memory(), x_host.clone().pin_memory()]
    lh = [logits_host.pin_memory(), logits_host.clone().pin_memory()]
    yh = [torch.empty(M_TOK, HID, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    xd = [torch.empty_like(x) for _ in range(2)]
    ld = [torch.empty_like(logits) for _ in range(2)]
    yd = [torch.empty_like(y) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    s_cmp = torch.cuda.current_stream()

    def e2e_loop(n):
        ev_in = [None, None]
        ev_cmp = [None, None]
        ev_out = [None, None]
        for i in range(n):
            b = i & 1
            if rank == 0:
                with torch.cuda.stream(s_in):
                    if ev_cmp[b] is not None:
                        s_in.wait_event(ev_cmp[b])           # x/logits buffer b is free again
                    xd[b].copy_(xh[b], non_blocking=True)
                    ld[b].copy_(lh[b], non_blocking=True)
                    ev_in[b] = torch.cuda.Event()
                    ev_in[b].record(s_in)
                s_cmp.wait_event(ev_in[b])
            if world > 1:
                # the inputs enter the node once, on rank 0, and reach the other ranks over NVLink
                dist.broadcast(xd[b], src=0)
                dist.broadcast(ld[b], src=0)
            if ev_out[b] is not None:
                s_cmp.wait_event(ev_out[b])              # y buffer b has been read back
            res = step(None, xd[b], ld[b], yd[b])
            if fused and rank == 0:
                yd[b].copy_(res)     # the shared output buffer is overwritten by the next step
            ev_cmp[b] = torch.cuda.Event()
            ev_cmp[b].record(s_cmp)
            if rank == 0:                                # the reduced result is identical on every rank
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[b])
                    yh[b].copy_(yd[b], non_blocking=True)
                    ev_out[b] = torch.cuda.Event()
                    ev_out[b].record(s_out)

    if not args.skip_e2e:
        e2e_loop(args.warmup)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        g0.record(s_in)
        e2e_loop(args.steps)
        s_out.synchronize()
        g1.record(s_out)
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3
        e2e_ms = max(g0.elapsed_time(g1), 0.0)
        if not (0.5 * wall_ms <= e2e_ms <= 1.5 * wall_ms):
            e2e_ms = wall_ms                     # events on two streams disagree with the host clock
        t = torch.tensor([e2e_ms], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms_step = float(t.item()) / args.steps
    h2d = x_host.numel() * 2 + logits_host.numel() * 4
    d2h = M_TOK * HID * 2

    # ---- dense cuBLAS equivalent (same run, same tensors) ------------------------------
    dense = None
    if world == 1 and not args.skip_dense:
        def dense_step():
            h = torch.nn.functional.silu(x @ wg.T) * (x @ wu.T)
            return h @ wd.T
        for _ in range(3):
            dense_step()
        torch.cuda.synchronize()
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0.record()
        for _ in range(args.steps):
            dense_step()
        d1.record()
        torch.cuda.synchronize()
        dms = d0.elapsed_time(d1) / args.steps
        dense = {"value": M_TOK / (dms * 1e-3), "unit": UNIT, "ms_per_step": dms,
                 "what": "torch.matmul x3 + silu*mul (cuBLAS bf16), all 112 groups"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak_tf, peak_gbs, peak_src = measured_peaks()
    # algorithmic flops of the fused gate/up GEMM: 2 weights * 2*H*G per active (token, group)
    flops_mn = 2 * 2.0 * HID * 128 * (M_TOK * KEEP) / world
    flops_k = 2.0 * HID * 128 * (M_TOK * KEEP) / world
    ach = flops_mn / (k_mn * 1e-3) / 1e12
    value = M_TOK / (ms_step * 1e-3)
    cpu = None if args.no_cpu_baseline or world > 1 else cpu_baseline()
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "parallelism": "single GPU" if world == 1 else
                   (f"tp{world} by channel groups ({gpr} groups per rank); the down projection stores "
                    "its partial token windows into the owning rank's memory (NVLink), a reduce+gather "
                    "kernel adds them and hands the rows to every rank; one-element all-reduces as "
                    f"barriers; tokens in {args.halves} part(s), the first part's gather under the second "
                    "part's projection" if fused else
                    f"tp{world} by channel groups ({gpr} groups per rank) + NCCL all-reduce of y in "
                    f"{chunks} token chunks overlapping the down projection, {args.sm_margin} SMs "
                    "left to the collective"),
                   "l2": "inputs larger than L2 (x 64 MiB + weights 336 MiB + h 224 MiB per step)",
                   "seed": SEED},
        "roofline": {"kernel": "gemm_mn_pair_kernel (fused gate/up + SwiGLU, CTA pairs)", "bound": "tensor",
                     "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s", "frac": ach / peak_tf,
                     "peak_source": f"{peak_src} sustained bf16",
                     # dram__bytes_read.sum + dram__bytes_write.sum of one full-size launch
                     # (profiles/gemm_kernels_config2_counters.md); scales with the rank's share
                     "traffic": (1.095717e9 + 1.186e8) / world if M_TOK == 8192 else None,
                     "traffic_source": "ncu capture of one launch at this size, see profiles/",
                     "algorithmic_flops_per_launch": flops_mn},
        "kernels": {"gemm_mn_ms": k_mn, "gemm_k_ms": k_k,
                    "gemm_k_ms_covers": ("down projection + barrier + reduce/gather + barrier" if fused
                                         else "down projection"),
                    "gemm_k_algorithmic_tflops": flops_k / (k_k * 1e-3) / 1e12,
                    "gemm_k_executed_tflops": 2.0 * flops_k / (k_k * 1e-3) / 1e12,
                    "other_ms": ms_step - k_mn - k_k},
        "clocks": clocks,
        "e2e": None if e2e_ms_step is None else {
            "value": M_TOK / (e2e_ms_step * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms_step,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "how": "pinned host x+logits -> device (rank 0, then NVLink broadcast when N > 1), "
                   "routed FFN, y -> pinned host (rank 0); double buffered over 3 streams"},
        "gpu_launches": launches_per_step * args.steps,
    }
    if dense is not None:
        out["dense"] = dense
        out["speedup_vs_dense"] = value / dense["value"]
    if cpu is not None:
        out["cpu_baseline"] = cpu
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
