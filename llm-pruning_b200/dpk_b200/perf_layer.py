"""Throughput of the Llama-3-70B-shaped pruned decoder layer (BASELINE config 5),
tensor-parallel over the ranks of one node.

    python -m dpk_b200.perf_layer                                   # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 \
        --master-addr 127.0.0.1 --master-port 29511 -m dpk_b200.perf_layer

hidden 8192, intermediate 28672 as 224 groups of 128 (top-112 per token), 64 query /
8 KV heads of dimension 128 (top-6 of 8 head groups per token), 16384-token prefill,
bf16, synthetic seeded tensors.  Rank r owns 8/N KV-head groups and 224/N channel
groups; the partial outputs of the output and down projections are all-reduced
(NCCL).  Prints one JSON line on rank 0: tokens/s, ms, phase split, roofline fraction.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from . import ops, tp
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
    ga0, ga1 = tp.group_range(NGA, world, rank)
    gf0, gf1 = tp.group_range(NGF, world, rank)
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

    def step():
        am = ops.topk_route_mask(la, KEEPA)[..., ga0:ga1]
        fm = ops.topk_route_mask(lf, KEEPF)[..., gf0:gf1]
        return layer(x, am, fm)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    layer.timers = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    status = ops.device_status()
    if status:
        raise SystemExit(f"a kernel reported status {status}")
    names = ["start", "qkv", "attn", "oproj", "ar1", "ffn", "ar2"]
    phases = {}
    tm = layer.timers
    for a, b in zip(names[:-1], names[1:]):
        phases[b + "_ms"] = sum(x0.elapsed_time(x1) for x0, x1 in zip(tm[a], tm[b])) / len(tm[a])
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
            "n_gpus": world, "parallelism": f"tp{world}: {hk_l} KV-head groups and {gf1 - gf0} "
            "channel groups per rank, 2 NCCL all-reduces of [T,H] bf16",
            "ms_per_layer": ms, "tokens_per_s": T / (ms * 1e-3), "phases": phases,
            "algorithmic_tflop": flops / 1e12,
            "roofline": {"bound": "tensor", "achieved": ach, "peak": peak_tf * world,
                         "unit": "TFLOP/s", "frac": ach / (peak_tf * world),
                         "peak_source": src + f" sustained bf16 x {world} GPUs"},
            "data": "synthetic, seed %d" % SEED}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
