"""Fused row-parallel sum on real peers (needs at least two GPUs; skipped otherwise).
Each rank is one process; the partial sums travel through mapped peer memory.  The result
is compared with the same partial sums added by an NCCL all-reduce and with the oracle."""

import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    sys.path[:0] = [ROOT, os.path.join(ROOT, "llm-pruning_b200")]
    import torch.distributed as dist
    from dpk_b200 import ops, tp
    from dpk_b200.ffn import RoutedFFN
    from dpk_b200.peer import RowParallelSum
    from oracle import dpk_oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        bf = torch.bfloat16
        g = torch.Generator().manual_seed(5)                  # replicated inputs
        M, H, I, NG = 2100, 512, 2048, 16
        x = torch.randn(1, M, H, generator=g).to(bf)
        wg = (torch.randn(I, H, generator=g) * 0.05).to(bf)
        wu = (torch.randn(I, H, generator=g) * 0.05).to(bf)
        wd = (torch.randn(H, I, generator=g) * 0.05).to(bf)
        mask = O.topk_route_mask(torch.randn(1, M, NG, generator=g), NG // 2)
        lg, lu, ld = (t.to(dev) for t in tp.shard_ffn_weights(wg, wu, wd, NG, world, rank))
        lmask = tp.shard_mask(mask, world, rank).to(dev)
        ffn = RoutedFFN(lg, lu, ld, NG // world, M)
        xd = x.to(dev)
        y_nccl = ffn(xd, lmask).clone()
        dist.all_reduce(y_nccl)
        y_nccl = y_nccl + xd
        ffn.row_parallel = RowParallelSum.connect(M, H, bf, dev)
        for _ in range(3):                                    # buffers are reused call after call
            y = ffn(xd, lmask, residual=xd)
        torch.cuda.synchronize()
        y_one = y.clone()
        ffn.row_parallel.halves = 2                           # overlapped schedule, second stream
        for _ in range(3):
            y = ffn(xd, lmask, residual=xd)
        torch.cuda.synchronize()
        # the same schedule with the barriers as flags in peer memory instead of NCCL all-reduces
        ffn.row_parallel.barrier_mode = "flags"
        for _ in range(4):
            y_flags = ffn(xd, lmask, residual=xd)
        torch.cuda.synchronize()
        flags_equal = bool(torch.equal(y_flags, y_one))
        ffn.row_parallel.barrier_mode = "nccl"
        y = ffn(xd, lmask, residual=xd)
        torch.cuda.synchronize()
        want = x.float() + O.ffn_swiglu(x.float(), wg.float(), wu.float(), wd.float(), mask,
                                        round_intermediate=bf)
        ret[rank] = dict(
            flags_equal=flags_equal,
            vs_nccl=O.rel_err(y.float().cpu(), y_nccl.float().cpu()),
            vs_oracle=O.rel_err(y.float().cpu(), want),
            halves_equal=bool(torch.equal(y, y_one)),
            status=ops.device_status(),
            digest=float(y.float().sum().item()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_row_parallel_ffn_two_ranks():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        out = dict(ret)
    assert sorted(out) == list(range(world))
    for r in range(world):
        assert out[r]["status"] == 0
        assert out[r]["halves_equal"]          # same slabs summed in the same order: same bits
        assert out[r]["flags_equal"]           # ... whichever barrier separates the two kernels
        assert out[r]["vs_oracle"] <= 2e-2, out[r]
        # one rounding of the sum instead of one per partial and one for the residual
        assert out[r]["vs_nccl"] <= 2e-2, out[r]
    assert out[0]["digest"] == out[1]["digest"]       # both ranks hold the same bits


def _layer_worker(rank, world, port, ret):
    sys.path[:0] = [ROOT, os.path.join(ROOT, "llm-pruning_b200")]
    import torch.distributed as dist
    from dpk_b200 import ops, tp
    from dpk_b200.layer import RoutedDecoderLayer
    from oracle import dpk_oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        bf = torch.bfloat16
        r16 = lambda t: t.to(bf).float()
        g = torch.Generator().manual_seed(9)                  # replicated inputs and weights
        T, H, Hq, Hk, D, I, NGF = 1100, 256, 8, 2, 64, 1024, 8
        ws = {n: r16(torch.randn(*shp, generator=g) * 0.05) for n, shp in dict(
            wq=(Hq * D, H), wk=(Hk * D, H), wv=(Hk * D, H), wo=(H, Hq * D),
            wg=(I, H), wu=(I, H), wd=(H, I)).items()}
        x = r16(torch.randn(1, T, H, generator=g))
        am = torch.rand(1, T, Hk, generator=g) > 0.3
        fm = O.topk_route_mask(torch.randn(1, T, NGF, generator=g), 4)
        lq, lk, lv, lo = tp.shard_attention(ws["wq"], ws["wk"], ws["wv"], ws["wo"], Hq, Hk, D, world, rank)
        lg, lu, ld = tp.shard_ffn_weights(ws["wg"], ws["wu"], ws["wd"], NGF, world, rank)
        d = lambda t: t.to(dev, bf)
        layer = RoutedDecoderLayer(d(lq), d(lk), d(lv), d(lo), d(lg), d(lu), d(ld),
                                   num_q_heads=Hq // world, num_kv_heads=Hk // world, head_dim=D,
                                   attn_groups=Hk // world, ffn_groups=NGF // world, max_tokens=T)
        lam, lfm = tp.shard_mask(am, world, rank).to(dev), tp.shard_mask(fm, world, rank).to(dev)
        out_nccl = layer(d(x), lam, lfm).clone()              # two NCCL all-reduces
        layer.fuse_sums(T)
        layer.sum_o.halves = layer.ffn.row_parallel.halves = 2
        out_fused = layer(d(x), lam, lfm).clone()
        torch.cuda.synchronize()
        q = r16(O.gemm_mn(x, ws["wq"], am)).view(1, T, Hq, D)
        k = r16(x @ ws["wk"].T).view(1, T, Hk, D)
        v = r16(x @ ws["wv"].T).view(1, T, Hk, D)
        a = r16(O.attention_prefill(q, k, v, am)).view(1, T, Hq * D)
        x1 = r16(x + r16(O.gemm_k(a, ws["wo"], am)))
        want = x1 + O.ffn_swiglu(x1, ws["wg"], ws["wu"], ws["wd"], fm, round_intermediate=bf)
        ret[rank] = dict(nccl=O.rel_err(out_nccl.float().cpu(), want),
                         fused=O.rel_err(out_fused.float().cpu(), want),
                         status=ops.device_status())
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_layer_matches_single_rank_oracle():
    """The tp=2 layer (KV-head groups and channel groups split, both ways of summing the partial
    outputs) against the oracle's unsplit composition."""
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_layer_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        out = dict(ret)
    for r in range(world):
        assert out[r]["status"] == 0
        assert out[r]["nccl"] <= 3e-2 and out[r]["fused"] <= 3e-2, out[r]
