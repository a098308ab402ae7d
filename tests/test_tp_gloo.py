"""Tensor-parallel host logic on two CPU ranks (gloo).  The per-rank compute is the
CPU oracle, so this checks the partitioning and the exchange step, not the kernels."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dpk_b200 import tp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "llm-pruning_b200")]
    from oracle import dpk_oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(3)              # same seed: replicated inputs
        B, T, H, I, NG = 2, 40, 64, 512, 8
        x = torch.randn(B, T, H, generator=g)
        wg, wu = torch.randn(I, H, generator=g) * 0.1, torch.randn(I, H, generator=g) * 0.1
        wd = torch.randn(H, I, generator=g) * 0.1
        mask = O.topk_route_mask(torch.randn(B, T, NG, generator=g), 3)
        lg, lu, ld = tp.shard_ffn_weights(wg, wu, wd, NG, world, rank)
        ffn = tp.TensorParallelFFN(lambda xx, mm: O.ffn_swiglu(xx, lg, lu, ld, mm), NG)
        y = ffn(x, mask)
        want = O.ffn_swiglu(x, wg, wu, wd, mask)
        ok_ffn = torch.allclose(y, want, atol=1e-4, rtol=1e-4)

        # attention by KV-head groups + row-parallel output projection
        Hq, Hk, D = 8, 4, 16
        q = torch.randn(B, T, Hq, D, generator=g)
        k, v = torch.randn(B, T, Hk, D, generator=g), torch.randn(B, T, Hk, D, generator=g)
        wo = torch.randn(H, Hq * D, generator=g) * 0.1
        am = torch.rand(B, T, Hk, generator=g) > 0.4
        k0, k1 = tp.group_range(Hk, world, rank)
        rep = Hq // Hk
        o_local = O.attention_prefill(q[:, :, k0 * rep:k1 * rep], k[:, :, k0:k1], v[:, :, k0:k1],
                                      tp.shard_mask(am, world, rank))
        part = o_local.flatten(2) @ wo[:, k0 * rep * D:k1 * rep * D].T
        dist.all_reduce(part)
        want_o = O.attention_prefill(q, k, v, am).flatten(2) @ wo.T
        ok_attn = torch.allclose(part, want_o, atol=1e-4, rtol=1e-4)
        # the fused row-parallel sum's data movement (owner blocks of whole 128-token windows,
        # contributions added in rank order, finished rows to everyone) as point-to-point messages
        Mrows = 300
        part2 = torch.randn(Mrows, H, generator=torch.Generator().manual_seed(11 + rank)).to(torch.bfloat16)
        res2 = torch.randn(Mrows, H, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
        summed = tp.owner_block_sum(part2, residual=res2)
        total = part2.float().clone()
        dist.all_reduce(total)
        want_sum = (total + res2.float()).to(torch.bfloat16)
        ok_sum = torch.equal(summed, want_sum)
        ret[rank] = (ok_ffn, ok_attn, ok_sum)
    finally:
        dist.destroy_process_group()


def test_two_rank_partition_and_allreduce():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}


def test_partition_helpers():
    assert tp.group_range(112, 8, 3) == (42, 56)
    with pytest.raises(ValueError):
        tp.group_range(112, 5, 0)
    with pytest.raises(ValueError):
        tp.group_range(8, 2, 2)
    g = torch.arange(6 * 4, dtype=torch.float32).reshape(6, 4)
    lg, lu, ld = tp.shard_ffn_weights(g, g + 100, g.T.contiguous(), 3, 3, 1)
    assert torch.equal(lg, g[2:4]) and torch.equal(lu, g[2:4] + 100)
    assert torch.equal(ld, g.T[:, 2:4])
    m = torch.arange(8).reshape(1, 8)
    assert torch.equal(tp.shard_mask(m, 4, 2), m[:, 4:6])
    wq = torch.arange(8 * 2 * 3, dtype=torch.float32).reshape(16, 3)      # Hq=8, D=2
    wk = torch.arange(4 * 2 * 3, dtype=torch.float32).reshape(8, 3)       # Hk=4
    q, k, v, o = tp.shard_attention(wq, wk, wk, wq.T.contiguous(), 8, 4, 2, 2, 1)
    assert torch.equal(q, wq[8:16]) and torch.equal(k, wk[4:8]) and torch.equal(o, wq.T[:, 8:16])
