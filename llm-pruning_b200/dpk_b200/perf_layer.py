"""Throughput of the Llama-3-70B-shaped pruned decoder layer (the tensor-parallel benchmark case),
tensor-parallel over the ranks of one node.

    python -m dpk_b200.perf_layer                                   # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 \
        --master-addr 127.0.0.1 --master-port 29511 -m dpk_b200.perf_layer

hidden 8192, intermediate 28672 as 224 groups of 128 (top-112 per token), 64 query /
8 KV heads of dimension 128 (top-6 of 8 head groups per token), 16384-token prefill,
bf16, synthetic seeded tensors.  Rank r owns 8/N KV-head groups and 224/N channel
groups; the partial outputs of the output and down projections are all-reduced
(NCCL).  Prints one JSON line on rank 0: tokens/s, ms, phase split, roofline fraction,
and the same layer without routing (cuBLAS projections, SDPA attention, the same
sharding and all-reduces) timed in the same run.

``--token-chunks C`` (N > 1) runs the layer as a pipeline over C chunks of query rows so
that the all-reduces overlap compute; ``--sm-margin S`` keeps S SMs free of the
persistent kernels for the collective.  ``--sweep "C:S,C:S,..."`` times several such
settings in one process and reports the best, with every setting's time listed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from . import _native, ops, tp
from .layer import RoutedDecoderLayer
from .perf import peaks

H, I, HQ, HK, D = 8192, 28672, 64, 8, 128
NGF, KEEPF, NGA, KEEPA = 224, 112, 8, 6
SEED = 17


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--token-chunks", type=int, default=0,
                    help="0 = automatic: 4 when N > 1, else 1")
    ap.add_argument("--sm-margin", type=int, default=-1, help="-1 = automatic: 8 when chunked")
    ap.add_argument("--sweep", default="", help='e.g. "1:0,2:8,4:8,4:16"')
    ap.add_argument("--skip-dense", action="store_true")
    ap.add_argument("--full", action="store_true",
                    help="include what surrounds the operators in the reference's layer: the two "
                         "token routers with their decisions, both RMSNorms and the rotary embedding "
                         "(the routing then comes from the routers, not from a top-k of given logits)")
    ap.add_argument("--halves", type=int, default=2, choices=[1, 2],
                    help="fused sums: 2 = project the tokens in two halves and gather the first "
                         "half under the second half's projection")
    ap.add_argument("--nccl-sums", action="store_true",
                    help="N > 1: sum the partial outputs with NCCL all-reduces instead of the "
                         "fused row-parallel sums")
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="single process: time rank 0's share of a W-way split (its shapes, "
                         "its kernels, no collective)")
    args = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T = args.tokens
    bf = torch.bfloat16
    split = args.emulate_world if (args.emulate_world > 0 and world == 1) else world
    ga0, ga1 = tp.group_range(NGA, split, rank)
    gf0, gf1 = tp.group_range(NGF, split, rank)
    hk_l, hq_l, i_l = ga1 - ga0, (ga1 - ga0) * (HQ // HK), (gf1 - gf0) * 128
    # this rank's weight slices, drawn directly in their sharded shapes
    gw = torch.Generator(device=dev).manual_seed(SEED + 1 + rank)

    def w(rows, cols):
        return (torch.randn(rows, cols, generator=gw, device=dev) * 0.02).to(bf)

    layer = RoutedDecoderLayer(w(hq_l * D, H), w(hk_l * D, H), w(hk_l * D, H), w(H, hq_l * D),
                               w(i_l, H), w(i_l, H), w(H, i_l), num_q_heads=hq_l,
                               num_kv_heads=hk_l, head_dim=D, attn_groups=hk_l,
                               ffn_groups=gf1 - gf0, max_tokens=T)
    # replicated inputs and router logits: same seed on every rank
    gx = torch.Generator(device=dev).manual_seed(SEED)
    x = torch.randn(1, T, H, generator=gx, device=dev).to(bf)
    la = torch.randn(1, T, NGA, generator=gx, device=dev)
    lf = torch.randn(1, T, NGF, generator=gx, device=dev)

    if args.full:
        R = 16
        def router(ng, keep_frac):
            wdn = (torch.randn(R, H, generator=gx, device=dev) / H ** 0.5).to(bf)
            wrt = (torch.randn(2 * ng, R, generator=gx, device=dev) / R ** 0.5).to(bf)
            brt = torch.zeros(2 * ng, device=dev)
            # logits of a pair differ by N(0, 2): shift the "execute" logit to the wanted quantile
            brt[0::2] = 2 ** 0.5 * torch.distributions.Normal(0.0, 1.0).icdf(torch.tensor(keep_frac)).item()
            return wdn, torch.zeros(R, device=dev).to(bf), wrt, brt.to(bf)
        n1 = (1.0 + 0.1 * torch.randn(H, generator=gx, device=dev)).to(bf)
        n2 = (1.0 + 0.1 * torch.randn(H, generator=gx, device=dev)).to(bf)
        layer.set_front_end(router(NGA, KEEPA / NGA), router(NGF, KEEPF / NGF), n1, n2, 1e-5,
                            (ga0, ga1), (gf0, gf1))
        inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=dev).float() / D))
        ang = torch.arange(T, device=dev).float()[:, None] * inv[None, :]
        cos, sin = torch.cat([ang, ang], -1).cos().to(bf), torch.cat([ang, ang], -1).sin().to(bf)

    def step():
        if args.full:
            return layer.forward_full(x, cos, sin)
        am = ops.topk_route_mask(la, KEEPA)[..., ga0:ga1]
        fm = ops.topk_route_mask(lf, KEEPF)[..., gf0:gf1]
        return layer(x, am, fm)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.sweep:
        settings = [tuple(int(v) for v in item.split(":")) for item in args.sweep.split(",")]
    else:
        chunks = args.token_chunks if args.token_chunks > 0 else (4 if world > 1 else 1)
        margin = args.sm_margin if args.sm_margin >= 0 else (8 if chunks > 1 and world > 1 else 0)
        settings = [(chunks, margin)]
    lib = _native.load()
    fused = world > 1 and not args.nccl_sums
    nccl_ms = None
    if fused:
        # the all-reduce schedule first, for the comparison; then switch the layer over
        layer.token_chunks = 1
        nccl_ms = timed(step)
        layer.fuse_sums(T)
        layer.sum_o.halves = layer.ffn.row_parallel.halves = args.halves
        settings = [(1, 0)]
    tried = {}
    for chunks, margin in settings:
        _native.check(lib.dpk_set_sm_margin(margin))
        layer.token_chunks = chunks
        tried[f"{chunks}:{margin}"] = timed(step)
    best = min(tried, key=tried.get)
    ms = tried[best]
    chunks, margin = (int(v) for v in best.split(":"))

    fused_phases = None
    if fused:
        layer.sum_o.timers, layer.ffn.row_parallel.timers = {}, {}
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        fused_phases = {"o_projection": layer.sum_o.phase_ms(),
                        "down_projection": layer.ffn.row_parallel.phase_ms()}
        layer.sum_o.timers, layer.ffn.row_parallel.timers = None, None

    # phase split: the unpipelined schedule, one phase after the other
    _native.check(lib.dpk_set_sm_margin(0))
    layer.token_chunks = 1
    sums = (layer.sum_o, layer.ffn.row_parallel)
    layer.sum_o, layer.ffn.row_parallel = None, None      # phases of the all-reduce schedule
    layer.timers = {}
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    names = (["start", "route1", "qkv", "attn", "oproj", "route2", "ffn"] if args.full else
             ["start", "qkv", "attn", "oproj", "ar1", "ffn", "ar2"])
    phases = {}
    tm = layer.timers
    for a, b in zip(names[:-1], names[1:]):
        phases[b + "_ms"] = sum(x0.elapsed_time(x1) for x0, x1 in zip(tm[a], tm[b])) / len(tm[a])
    layer.timers = None
    layer.sum_o, layer.ffn.row_parallel = sums
    status = ops.device_status()
    if status:
        raise SystemExit(f"a kernel reported status {status}")

    dense_ms = None
    if not args.skip_dense:
        wq, wk, wv, wo = layer.wq, layer.wk, layer.wv, layer.wo
        wg, wu, wd = layer.ffn.wg, layer.ffn.wu, layer.ffn.wd
        sdpa = torch.nn.functional.scaled_dot_product_attention

        def rot(t):
            half = D // 2
            return t * cos[None, :, None, :] + torch.cat((-t[..., half:], t[..., :half]), -1) * sin[None, :, None, :]

        def dense_step():
            xf = x[0]
            if args.full:
                xn = torch.nn.functional.rms_norm(xf, (H,), n1, 1e-5)
                q = rot((xn @ wq.T).view(1, T, hq_l, D)).transpose(1, 2)
                k = rot((xn @ wk.T).view(1, T, hk_l, D)).transpose(1, 2)
                v = (xn @ wv.T).view(1, T, hk_l, D).transpose(1, 2)
                a = sdpa(q, k, v, is_causal=True, enable_gqa=True).transpose(1, 2).reshape(T, hq_l * D)
                o = a @ wo.T
                if world > 1:
                    dist.all_reduce(o)
                x1 = xf + o
                x1n = torch.nn.functional.rms_norm(x1, (H,), n2, 1e-5)
                yy = (torch.nn.functional.silu(x1n @ wg.T) * (x1n @ wu.T)) @ wd.T
                if world > 1:
                    dist.all_reduce(yy)
                return x1 + yy
            q = (xf @ wq.T).view(1, T, hq_l, D).transpose(1, 2)
            k = (xf @ wk.T).view(1, T, hk_l, D).transpose(1, 2)
            v = (xf @ wv.T).view(1, T, hk_l, D).transpose(1, 2)
            a = sdpa(q, k, v, is_causal=True, enable_gqa=True).transpose(1, 2).reshape(T, hq_l * D)
            o = a @ wo.T
            if world > 1:
                dist.all_reduce(o)
            x1 = xf + o
            hmid = torch.nn.functional.silu(x1 @ wg.T) * (x1 @ wu.T)
            yy = hmid @ wd.T
            if world > 1:
                dist.all_reduce(yy)
            return x1 + yy

        dense_ms = timed(dense_step)
    if rank == 0:
        peak_tf, _, src = peaks()
        # algorithmic flops of the whole layer (all ranks)
        pairs_attn = KEEPA / NGA * HQ * (T * (T + 1) / 2)
        flops = (6.0 * H * 128 * T * KEEPF          # FFN
                 + 4.0 * D * pairs_attn             # attention
                 + 2.0 * H * (HQ // NGA) * D * T * KEEPA * 2    # Q and O projections
                 + 2.0 * 2 * H * HK * D * T)        # dense K, V projections
        ach = flops / (ms * 1e-3) / 1e12
        print(json.dumps({
            "workload": f"llama3-70b-shaped pruned layer: H={H} I={I} ({NGF}x128, top-{KEEPF}) "
                        f"Hq={HQ} Hk={HK} D={D} (top-{KEEPA} of {NGA} head groups) tokens={T}",
            "n_gpus": world, "parallelism": f"tp{split}{' (rank 0 alone, no collective)' if split != world else ''}: {hk_l} KV-head groups and {gf1 - gf0} "
            "channel groups per rank, " + (
                "row-parallel sums fused into the o and down projections (stores into the owning "
                f"rank's memory, reduce + gather kernel, tokens in {args.halves} part(s))" if fused else
                f"2 NCCL all-reduces of [T,H] bf16, {chunks} token chunks pipelined, {margin} SMs "
                "left to the collective"),
            "ms_per_layer_with_nccl_all_reduce": nccl_ms,
            "fused_sum_phases_ms": fused_phases,
            "ms_per_layer": ms, "tokens_per_s": T / (ms * 1e-3),
            "settings_ms (chunks:sm_margin)": tried,
            "phases_unpipelined": phases,
            "dense_layer_ms": dense_ms,
            "speedup_vs_dense_layer": (dense_ms / ms) if dense_ms else None,
            "algorithmic_tflop": flops / 1e12,
            "roofline": {"bound": "tensor", "achieved": ach, "peak": peak_tf * world,
                         "unit": "TFLOP/s", "frac": ach / (peak_tf * world),
                         "peak_source": src + f" sustained bf16 x {world} GPUs"},
            "full_layer": bool(args.full),
            "data": "synthetic, seed %d" % SEED}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
