"""Throughput runner for the individual operator families.

Counterpart of the reference's ``run.py --run-type run_throughput``
(``DynamicPruningKernels/run.py:283-311``; metric definitions
``python/gemm_mn/jit.py:619-652``, ``python/attention_prefill/jit.py:538-541``): times a
family on seeded synthetic tensors with CUDA events, next to the dense PyTorch
equivalent (cuBLAS / SDPA), and prints one JSON line per case with the achieved rate
and its fraction of the measured roofline.

    python -m dpk_b200.perf --kernel attention_prefill      # 8192-token routed prefill attention
    python -m dpk_b200.perf --kernel attention_decode       # decode step, batch 64, 32768-token KV cache
    python -m dpk_b200.perf --kernel ffn_decode             # decode-step FFN, 64 tokens
    python -m dpk_b200.perf --kernel gemm_mn | gemm_k | ffn # Llama-3-8B-shaped FFN prefill and its two GEMMs
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

from . import _native, ops
from .ffn import RoutedFFN

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
SEED = 17


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("bf16_tflops_sustained", 1425.8), d.get("hbm_gbs", 6449.1), "measured"
    return 1400.0, 6650.0, "fallback"


def time_ms(fn, reps: int, warmup: int = 3):
    """Median and 20/80 % quantiles of per-call device time (CUDA events)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        samples.append(a.elapsed_time(b))
    samples.sort()
    q = lambda f: samples[min(len(samples) - 1, int(f * len(samples)))]
    return statistics.median(samples), q(0.2), q(0.8)


def topk_mask(shape, keep, gen):
    logits = torch.randn(*shape, generator=gen, device="cuda")
    return ops.topk_route_mask(logits, keep)


def run_prefill(args):
    B, T, Hq, Hk, D, NG, keep = 1, args.tokens or 8192, 32, 8, 128, 8, 4
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    bf = torch.float16 if getattr(args, "fp16", False) else torch.bfloat16
    q = torch.randn(B, T, Hq, D, generator=gen, device="cuda").to(bf)
    k = torch.randn(B, T, Hk, D, generator=gen, device="cuda").to(bf)
    v = torch.randn(B, T, Hk, D, generator=gen, device="cuda").to(bf)
    mask = topk_mask((B, T, NG), keep, gen)
    out = torch.zeros_like(q)
    ms, lo, hi = time_ms(lambda: ops.attention_prefill(q, k, v, mask, O=out), args.reps)
    # algorithmic flops: 4*D per (active query row, visible key) pair and query head
    pos = torch.arange(1, T + 1, device="cuda", dtype=torch.float64)
    pairs = float((mask.to(torch.float64) * pos[None, :, None]).sum()) * (Hq // NG)
    flops = 4.0 * D * pairs
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    dms, _, _ = time_ms(lambda: torch.nn.functional.scaled_dot_product_attention(
        qt, kt, vt, is_causal=True, enable_gqa=True), args.reps)
    peak_tf, _, src = peaks()
    ach = flops / (ms * 1e-3) / 1e12
    return {"kernel": "attention_prefill", "workload": f"B={B} T={T} Hq={Hq} Hk={Hk} D={D} causal, "
            f"top-{keep} of {NG} head groups", "ms": ms, "ms_q20": lo, "ms_q80": hi,
            "tokens_per_s": B * T / (ms * 1e-3), "algorithmic_tflops": flops / 1e12,
            "roofline": {"bound": "tensor", "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": ach / peak_tf, "peak_source": src + " sustained bf16"},
            "dense_sdpa_ms": dms, "speedup_vs_dense": dms / ms}


def run_decode(args):
    B, Tk, Hq, Hk, D, NG, keep = args.batch or 64, args.tokens or 32768, 32, 8, 128, 8, 4
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    bf = torch.bfloat16
    q = torch.randn(B, 1, Hq, D, generator=gen, device="cuda").to(bf)
    k = torch.randn(B, Tk, Hk, D, generator=gen, device="cuda", dtype=bf)
    v = torch.randn(B, Tk, Hk, D, generator=gen, device="cuda", dtype=bf)
    mask = topk_mask((B, 1, NG), keep, gen)
    out = torch.empty_like(q)
    ms, lo, hi = time_ms(lambda: ops.attention_decode(q, k, v, mask, O=out), args.reps)
    active_pairs = int(mask.sum())          # NG == Hk: one group per KV head
    nbytes = 2.0 * Tk * D * 2 * active_pairs
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    dms, _, _ = time_ms(lambda: torch.nn.functional.scaled_dot_product_attention(
        qt, kt, vt, is_causal=False, enable_gqa=True), max(3, args.reps // 4))
    _, peak_gbs, src = peaks()
    ach = nbytes / (ms * 1e-3) / 1e9
    return {"kernel": "attention_decode", "workload": f"B={B} Tk={Tk} Hq={Hq} Hk={Hk} D={D}, "
            f"top-{keep} of {NG} head groups, KV cache {2 * k.numel() * 2 / 2**30:.1f} GiB (> L2)",
            "tpot_us": ms * 1e3, "ms_q20": lo, "ms_q80": hi, "algorithmic_gbytes": nbytes / 1e9,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak_gbs, "unit": "GB/s",
                         "frac": ach / peak_gbs, "peak_source": src + " copy bandwidth"},
            "dense_sdpa_us": dms * 1e3, "speedup_vs_dense": dms / ms}


def _ffn_tensors(M, gen, H=4096, I=14336):
    bf = torch.bfloat16
    x = torch.randn(1, M, H, generator=gen, device="cuda").to(bf)
    wg = (torch.randn(I, H, generator=gen, device="cuda") * 0.02).to(bf)
    wu = (torch.randn(I, H, generator=gen, device="cuda") * 0.02).to(bf)
    wd = (torch.randn(H, I, generator=gen, device="cuda") * 0.02).to(bf)
    return x, wg, wu, wd


def run_ffn(args, decode=False):
    M = args.tokens or (64 if decode else 8192)
    H, I, NG, keep = 4096, 14336, 112, 56
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    x, wg, wu, wd = _ffn_tensors(M, gen, H, I)
    mask = topk_mask((1, M, NG), keep, gen)
    ffn = RoutedFFN(wg, wu, wd, NG, M)
    y = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    ms, lo, hi = time_ms(lambda: ffn(x, mask, out=y), args.reps)
    dms, _, _ = time_ms(lambda: (torch.nn.functional.silu(x @ wg.T) * (x @ wu.T)) @ wd.T, args.reps)
    peak_tf, peak_gbs, src = peaks()
    flops = 6.0 * H * 128 * M * keep
    used = int(mask.any(dim=1).sum())                      # groups some token uses
    wbytes = 3.0 * H * 128 * 2 * used
    res = {"kernel": "ffn_decode" if decode else "ffn", "workload": f"M={M} H={H} I={I} "
           f"NG={NG}x128 top-{keep}", "ms": ms, "ms_q20": lo, "ms_q80": hi,
           "tokens_per_s": M / (ms * 1e-3), "dense_ms": dms, "speedup_vs_dense": dms / ms}
    if decode:
        ach = wbytes / (ms * 1e-3) / 1e9
        res["roofline"] = {"bound": "hbm", "achieved": ach, "peak": peak_gbs, "unit": "GB/s",
                           "frac": ach / peak_gbs, "peak_source": src + " copy bandwidth",
                           "algorithmic_bytes": wbytes}
    else:
        ach = flops / (ms * 1e-3) / 1e12
        res["roofline"] = {"bound": "tensor", "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s",
                           "frac": ach / peak_tf, "peak_source": src + " sustained bf16"}
    return res


def run_gemm(args, which):
    if args.config == 5:      # the FFN of the 70B-shaped layer
        M, H, I, NG, keep = args.tokens or 16384, 8192, 28672, 224, 112
    else:
        M, H, I, NG, keep = args.tokens or 8192, 4096, 14336, 112, 56
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    x, wg, wu, wd = _ffn_tensors(M, gen, H, I)
    mask = topk_mask((1, M, NG), keep, gen)
    peak_tf, _, src = peaks()
    if which == "gemm_mn":
        out = torch.zeros(M, I, dtype=torch.bfloat16, device="cuda")
        _, meta = ops.gemm_mn(x, wg, mask)
        ms, lo, hi = time_ms(lambda: ops.gemm_mn(x, wg, mask, D=out, **meta), args.reps)
        dms, _, _ = time_ms(lambda: x @ wg.T, args.reps)
        flops = 2.0 * H * 128 * M * keep
    else:
        a = torch.randn(1, M, I, generator=gen, device="cuda").to(torch.bfloat16)
        out = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
        _, meta = ops.gemm_k(a, wd, mask)
        ms, lo, hi = time_ms(lambda: ops.gemm_k(a, wd, mask, D=out, **meta), args.reps)
        dms, _, _ = time_ms(lambda: a @ wd.T, args.reps)
        flops = 2.0 * H * 128 * M * keep
    # the native call alone (routing layout and packed bits prepared once, no Python shim)
    from . import _native as N
    lib, st = N.load(), torch.cuda.current_stream().cuda_stream
    if which == "gemm_mn":
        counts = ops._counts_of(meta["sorted_mask"])
        sidx = meta["sorted_indices"]
        xf = x.view(M, H)
        kms, _, _ = time_ms(lambda: N.check(lib.dpk_gemm_mn(
            xf.data_ptr(), H, wg.data_ptr(), None, H, sidx.data_ptr(), counts.data_ptr(),
            out.data_ptr(), I, M, I, H, NG, N.BF16, 0, st)), args.reps)
    else:
        words = (NG + 31) // 32
        rb = torch.empty((M, words), dtype=torch.int32, device="cuda")
        wb = torch.empty(((M + 127) // 128, words), dtype=torch.int32, device="cuda")
        m8 = mask.view(torch.uint8).view(M, NG)
        N.check(lib.dpk_mask_pack(m8.data_ptr(), M, NG, rb.data_ptr(), wb.data_ptr(), st))
        af = a.view(M, I)
        kms, _, _ = time_ms(lambda: N.check(lib.dpk_gemm_k(
            af.data_ptr(), I, wd.data_ptr(), I, rb.data_ptr(), wb.data_ptr(), out.data_ptr(), H,
            M, H, I, NG, N.BF16, None, 0, None, 0, st)), args.reps)
    ach = flops / (kms * 1e-3) / 1e12
    return {"kernel": which, "workload": f"M={M} H={H} I={I} NG={NG}x128 top-{keep}",
            "native_call_ms": kms, "ms": ms, "ms_q20": lo, "ms_q80": hi,
            "ms_is": "through the Python operator API with reused routing metadata",
            "dense_equiv_tflops": 2.0 * M * H * I / (ms * 1e-3) / 1e12,
            "roofline": {"bound": "tensor", "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": ach / peak_tf, "peak_source": src + " sustained bf16"},
            "dense_ms": dms, "speedup_vs_dense": dms / kms, "speedup_vs_dense_through_api": dms / ms}


def run_router_norm(args):
    """Router + RMSNorm in front of the 70B-shaped layer: H=8192, 224 FFN groups, rank 16."""
    M, H, NG, R = args.tokens or 16384, args.hidden or 8192, 224, 16
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    bf = torch.bfloat16
    x = torch.randn(M, H, generator=gen, device="cuda").to(bf)
    gamma = (1.0 + 0.1 * torch.randn(H, generator=gen, device="cuda")).to(bf)
    wd = (torch.randn(R, H, generator=gen, device="cuda") / H ** 0.5).to(bf)
    bd = (0.1 * torch.randn(R, generator=gen, device="cuda")).to(bf)
    wr = (torch.randn(2 * NG, R, generator=gen, device="cuda") / R ** 0.5).to(bf)
    br = (0.1 * torch.randn(2 * NG, generator=gen, device="cuda")).to(bf)
    # The kernel itself: twenty launches through the C ABI into preallocated outputs per sample.
    # The operator call adds the output allocations and the uint8 -> bool conversion of the
    # decisions (a second, small kernel); it is timed beside it, ten calls per sample.
    lib = _native.load()
    xn = torch.empty_like(x)
    execute = torch.empty(M, NG, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    def twenty():
        for _ in range(20):
            _native.check(lib.dpk_router_norm(x.data_ptr(), H, gamma.data_ptr(), 1e-5, wd.data_ptr(), bd.data_ptr(),
                                              wr.data_ptr(), br.data_ptr(), xn.data_ptr(), H, execute.data_ptr(),
                                              None, M, H, R, NG, _native.BF16, 1, stream))
    ms, lo, hi = (t / 20 for t in time_ms(twenty, args.reps))
    def ten():
        for _ in range(10):
            ops.router_norm(x, wd, bd, wr, br, norm_weight=gamma, eps=1e-5)
    api_ms = time_ms(ten, args.reps)[0] / 10

    def torch_equivalent():
        xf = x.float()
        xn = gamma * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(bf)
        logits = torch.nn.functional.linear(torch.nn.functional.linear(x, wd, bd), wr, br)
        return xn, logits.view(M, NG, 2).argmax(-1).bool().logical_not()

    def ten_torch():
        for _ in range(10):
            torch_equivalent()
    dms = time_ms(ten_torch, args.reps)[0] / 10
    nbytes = 2.0 * M * H * 2 + M * NG            # x read once, xn written once, decisions
    _, peak_gbs, src = peaks()
    ach = nbytes / (ms * 1e-3) / 1e9
    return {"kernel": "router_norm", "workload": f"M={M} H={H} NG={NG} rank={R}, RMSNorm output + "
            "decisions (x 256 MiB > L2)", "ms": ms, "ms_q20": lo, "ms_q80": hi, "operator_call_ms": api_ms,
            "algorithmic_bytes": nbytes,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak_gbs, "unit": "GB/s",
                         "frac": ach / peak_gbs, "peak_source": src + " copy bandwidth"},
            "torch_ms": dms, "speedup_vs_torch": dms / ms}


def run_gemm_k_scatter(args):
    """The tensor-parallel down projection of one rank (70B-shaped layer split 4 ways: 56 of 224
    channel groups) with its epilogue storing into the owners' staging slabs -- all four ranks'
    buffers live on this GPU (``RowParallelSum.emulate``), so the stores are local; what is
    measured is the kernel itself against the plain ``gemm_k`` on the same operands."""
    from .peer import RowParallelSum
    world, M, N, NG = 4, args.tokens or 8192, 8192, 56
    K = NG * 128
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    bf = torch.bfloat16
    a = torch.randn(M, K, generator=gen, device="cuda").to(bf)
    w = (torch.randn(N, K, generator=gen, device="cuda") * 0.02).to(bf)
    mask = topk_mask((1, M, NG), NG // 2, gen)[0]
    ranks = RowParallelSum.emulate(world, M, N, bf, torch.device("cuda"))
    words = (NG + 31) // 32
    rb = torch.empty((M, words), dtype=torch.int32, device="cuda")
    wb = torch.empty(((M + 127) // 128, words), dtype=torch.int32, device="cuda")
    m8 = mask.to(torch.uint8).contiguous()
    _native.check(_native.load().dpk_mask_pack(m8.data_ptr(), M, NG, rb.data_ptr(), wb.data_ptr(), None))
    ms, lo, hi = time_ms(lambda: ranks[1].scatter(a, w, rb, wb, NG), args.reps)
    d = torch.empty(1, M, N, dtype=bf, device="cuda")
    pms, _, _ = time_ms(lambda: ops.gemm_k(a[None], w, mask[None], D=d), args.reps)
    peak_tf, _, src = peaks()
    executed = 2.0 * N * K * M            # every window visits every group at a 50 % keep ratio
    ach = executed / (ms * 1e-3) / 1e12
    return {"kernel": "gemm_k_scatter", "workload": f"M={M} N={N} K={K} ({NG}x128, top-{NG // 2}), "
            f"rank 1 of {world} emulated on one GPU", "ms": ms, "ms_q20": lo, "ms_q80": hi,
            "plain_gemm_k_call_ms": pms,
            "roofline": {"bound": "tensor", "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": ach / peak_tf, "peak_source": src + " sustained bf16",
                         "note": "executed flops (the masked formulation runs 2x the algorithmic ones)"}}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--kernel", required=True,
                    choices=["attention_prefill", "attention_decode", "ffn", "ffn_decode",
                             "gemm_mn", "gemm_k", "router_norm", "gemm_k_scatter"])
    ap.add_argument("--hidden", type=int, default=0, help="override the hidden size (router_norm)")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=0, help="override the token / KV length")
    ap.add_argument("--batch", type=int, default=0, help="override the decode batch")
    ap.add_argument("--fp16", action="store_true", help="attention_prefill: fp16 tensors instead of bf16")
    ap.add_argument("--gather4", type=int, default=-1, choices=[-1, 0, 1],
                    help="gemm_mn / ffn: token rows by cp.async (0) or TMA tile::gather4 (1); -1 = the default")
    ap.add_argument("--heads-per-cta", type=int, default=0, choices=[0, 1, 2],
                    help="attention_prefill: 2 = the two-heads-per-CTA kernel, 0/1 = one head per CTA")
    ap.add_argument("--config", type=int, default=2, choices=[2, 5],
                    help="gemm_mn / gemm_k: FFN shape of BASELINE config 2 (4096/14336) or 5 (8192/28672)")
    ap.add_argument("--wave-order", type=int, default=1, choices=[0, 1],
                    help="gemm_k: 1 = grouped tile order with aligned waves where W exceeds L2, 0 = plain order")
    ap.add_argument("--router-cluster", type=int, default=1, choices=[0, 1],
                    help="router_norm: 1 = column-split cluster kernel where the width allows, 0 = one CTA per tile")
    args = ap.parse_args(argv)
    assert torch.cuda.is_available(), "dpk_b200.perf needs a CUDA device"
    _native.check(_native.load().dpk_set_router_norm_cluster(args.router_cluster))
    _native.check(_native.load().dpk_set_gemm_k_wave_order(args.wave_order))
    _native.check(_native.load().dpk_set_attn_prefill_heads(args.heads_per_cta))
    if args.gather4 >= 0:
        _native.check(_native.load().dpk_set_gemm_mn_gather(args.gather4))
    if args.kernel == "attention_prefill":
        res = run_prefill(args)
    elif args.kernel == "attention_decode":
        res = run_decode(args)
    elif args.kernel == "ffn":
        res = run_ffn(args)
    elif args.kernel == "ffn_decode":
        res = run_ffn(args, decode=True)
    elif args.kernel == "router_norm":
        res = run_router_norm(args)
    elif args.kernel == "gemm_k_scatter":
        res = run_gemm_k_scatter(args)
    else:
        res = run_gemm(args, args.kernel)
    status = ops.device_status()
    if status:
        raise SystemExit(f"a kernel reported status {status}")
    res["data"] = "synthetic, seed %d" % SEED
    print(json.dumps(res))


if __name__ == "__main__":
    sys.exit(main())
