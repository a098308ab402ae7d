"""Seeded synthetic tensors of the benchmark configurations.

The reference benchmarks its kernels on random tensors (``python/gemm_mn/jit.py:483-487``:
``randn`` activations, random masks, seed 17 from ``run.py:42``); the shapes and
distributions here are the ones the benchmark configurations state: activations, Q/K/V and
router logits N(0,1), weights N(0,0.02), all rounded to bf16 (logits stay fp32), top-k
routing.  Large tensors are drawn on the device with a seeded CUDA generator.  Every rank of
a tensor-parallel run draws the same full tensors and keeps its slice, so that the sharded
layer computes the same function as the single-GPU one.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from . import tp

SEED = 17
BF16 = torch.bfloat16


def _gen(dev, offset: int = 0) -> torch.Generator:
    return torch.Generator(device=dev).manual_seed(SEED + offset)


def _normal(gen, dev, *shape, std: float = 1.0, dtype=BF16) -> torch.Tensor:
    t = torch.randn(*shape, generator=gen, device=dev)
    if std != 1.0:
        t *= std
    return t.to(dtype)


# --------------------------------------------------------------------------- config 2

@dataclass(frozen=True)
class FfnShape:
    tokens: int = 8192
    hidden: int = 4096
    inter: int = 14336
    groups: int = 112
    keep: int = 56

    @property
    def name(self) -> str:
        return (f"llama3-8b-ffn-prefill: H={self.hidden} I={self.inter} NG={self.groups}x128 "
                f"tokens={self.tokens} top-{self.keep}")


def ffn_tensors(dev, shape: FfnShape = FfnShape()):
    """``x [1,M,H]``, ``wg, wu [I,H]``, ``wd [H,I]``, ``logits [1,M,NG]`` fp32."""
    g = _gen(dev)
    s = shape
    x = _normal(g, dev, 1, s.tokens, s.hidden)
    wg = _normal(g, dev, s.inter, s.hidden, std=0.02)
    wu = _normal(g, dev, s.inter, s.hidden, std=0.02)
    wd = _normal(g, dev, s.hidden, s.inter, std=0.02)
    logits = torch.randn(1, s.tokens, s.groups, generator=g, device=dev)
    return x, wg, wu, wd, logits


# --------------------------------------------------------------------------- config 3

@dataclass(frozen=True)
class PrefillShape:
    tokens: int = 8192
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    groups: int = 8
    keep: int = 4

    @property
    def name(self) -> str:
        return (f"routed-attention-prefill: {self.q_heads}q/{self.kv_heads}kv D={self.head_dim} "
                f"T={self.tokens} causal top-{self.keep} of {self.groups} head groups")


def prefill_tensors(dev, shape: PrefillShape = PrefillShape()):
    g = _gen(dev, 2)
    s = shape
    q = _normal(g, dev, 1, s.tokens, s.q_heads, s.head_dim)
    k = _normal(g, dev, 1, s.tokens, s.kv_heads, s.head_dim)
    v = _normal(g, dev, 1, s.tokens, s.kv_heads, s.head_dim)
    logits = torch.randn(1, s.tokens, s.groups, generator=g, device=dev)
    return q, k, v, logits


# --------------------------------------------------------------------------- config 4

@dataclass(frozen=True)
class DecodeShape:
    batch: int = 64
    kv_len: int = 32768
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    attn_groups: int = 8
    attn_keep: int = 4
    ffn: FfnShape = FfnShape(tokens=64)

    @property
    def name(self) -> str:
        return (f"decode-step: batch={self.batch} kv_len={self.kv_len} {self.q_heads}q/"
                f"{self.kv_heads}kv D={self.head_dim} top-{self.attn_keep} of {self.attn_groups} head "
                f"groups; FFN H={self.ffn.hidden} I={self.ffn.inter} top-{self.ffn.keep} of {self.ffn.groups}")


def decode_tensors(dev, shape: DecodeShape = DecodeShape()):
    """``q [B,1,Hq,D]``, ``k, v [B,Tk,Hk,D]`` (4 GiB each at full size), ``logits [B,1,NG]``."""
    g = _gen(dev, 3)
    s = shape
    q = _normal(g, dev, s.batch, 1, s.q_heads, s.head_dim)
    k = torch.empty(s.batch, s.kv_len, s.kv_heads, s.head_dim, dtype=BF16, device=dev)
    v = torch.empty_like(k)
    for t in (k, v):                      # per sequence: bounds the fp32 temporary
        for b in range(s.batch):
            t[b] = _normal(g, dev, s.kv_len, s.kv_heads, s.head_dim)
    logits = torch.randn(s.batch, 1, s.attn_groups, generator=g, device=dev)
    return q, k, v, logits


# --------------------------------------------------------------------------- config 5

@dataclass(frozen=True)
class LayerShape:
    tokens: int = 16384
    hidden: int = 8192
    inter: int = 28672
    q_heads: int = 64
    kv_heads: int = 8
    head_dim: int = 128
    attn_groups: int = 8
    attn_keep: int = 6
    ffn_groups: int = 224
    ffn_keep: int = 112
    router_rank: int = 16
    eps: float = 1e-5

    @property
    def name(self) -> str:
        return (f"llama3-70b-shaped pruned decoder layer: H={self.hidden} I={self.inter} "
                f"({self.ffn_groups}x128, {self.ffn_keep}/{self.ffn_groups} kept) Hq={self.q_heads} "
                f"Hk={self.kv_heads} D={self.head_dim} ({self.attn_keep}/{self.attn_groups} head "
                f"groups kept) tokens={self.tokens} prefill")

    def shard(self, world: int, rank: int) -> Tuple[Tuple[int, int], Tuple[int, int]]:
        return (tp.group_range(self.attn_groups, world, rank),
                tp.group_range(self.ffn_groups, world, rank))


WEIGHT_NAMES = ("wq", "wk", "wv", "wo", "wg", "wu", "wd")


def layer_weights(dev, shape: LayerShape, world: int = 1, rank: int = 0,
                  keep_host_fp32: bool = False):
    """This rank's weight slices of the layer and, with ``keep_host_fp32``, fp32 host copies of
    the FULL matrices (what a checker on the host needs).  Each full matrix is drawn on the
    device from the same seed on every rank, sliced, and released."""
    s = shape
    (ga0, ga1), (gf0, gf1) = s.shard(world, rank)
    hpg = s.q_heads // s.attn_groups * s.head_dim          # q channels per head group
    kpg = s.kv_heads // s.attn_groups * s.head_dim         # k/v channels per head group
    qd, kd = s.q_heads * s.head_dim, s.kv_heads * s.head_dim
    plan = {
        "wq": ((qd, s.hidden), 0, (ga0 * hpg, ga1 * hpg)),
        "wk": ((kd, s.hidden), 0, (ga0 * kpg, ga1 * kpg)),
        "wv": ((kd, s.hidden), 0, (ga0 * kpg, ga1 * kpg)),
        "wo": ((s.hidden, qd), 1, (ga0 * hpg, ga1 * hpg)),
        "wg": ((s.inter, s.hidden), 0, (gf0 * 128, gf1 * 128)),
        "wu": ((s.inter, s.hidden), 0, (gf0 * 128, gf1 * 128)),
        "wd": ((s.hidden, s.inter), 1, (gf0 * 128, gf1 * 128)),
    }
    g = _gen(dev, 1)
    mine: Dict[str, torch.Tensor] = {}
    host: Dict[str, torch.Tensor] = {}
    for name in WEIGHT_NAMES:
        full_shape, dim, (a, b) = plan[name]
        full = _normal(g, dev, *full_shape, std=0.02)
        mine[name] = (full[a:b] if dim == 0 else full[:, a:b]).contiguous()
        if keep_host_fp32:
            host[name] = full.float().cpu()
        del full
    return (mine, host) if keep_host_fp32 else mine


def layer_front_end(dev, shape: LayerShape):
    """Routers, norm weights and rotary tables of the layer (replicated on every rank).

    A router is ``(w_down [R,H], b_down [R], w_route [2*NG,R], b_route [2*NG])``; the bias of
    every group's "execute" logit is shifted so that the argmax decision keeps the
    configuration's fraction of groups on average (the two logits of a pair differ by N(0,2))."""
    s = shape
    g = _gen(dev, 4)
    H, R, D, T = s.hidden, s.router_rank, s.head_dim, s.tokens

    def router(ng: int, keep_fraction: float):
        w_down = _normal(g, dev, R, H, std=H ** -0.5)
        w_route = _normal(g, dev, 2 * ng, R, std=R ** -0.5)
        b_route = torch.zeros(2 * ng, device=dev)
        shift = 2 ** 0.5 * torch.distributions.Normal(0.0, 1.0).icdf(torch.tensor(keep_fraction)).item()
        b_route[0::2] = shift
        return w_down, torch.zeros(R, device=dev).to(BF16), w_route, b_route.to(BF16)

    attn_router = router(s.attn_groups, s.attn_keep / s.attn_groups)
    ffn_router = router(s.ffn_groups, s.ffn_keep / s.ffn_groups)
    n1 = (1.0 + 0.1 * torch.randn(H, generator=g, device=dev)).to(BF16)
    n2 = (1.0 + 0.1 * torch.randn(H, generator=g, device=dev)).to(BF16)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=dev).float() / D))
    ang = torch.arange(T, device=dev).float()[:, None] * inv[None, :]
    cos = torch.cat([ang, ang], -1).cos().to(BF16)
    sin = torch.cat([ang, ang], -1).sin().to(BF16)
    return dict(attn_router=attn_router, ffn_router=ffn_router, n1=n1, n2=n2, cos=cos, sin=sin)


def layer_input(dev, shape: LayerShape, host: bool = False) -> torch.Tensor:
    """The residual stream ``x [1,T,H]`` bf16 N(0,1); ``host=True`` draws it in (pageable) host
    memory from a CPU generator of the same seed."""
    if host:
        g = torch.Generator().manual_seed(SEED)
        return torch.randn(1, shape.tokens, shape.hidden, generator=g).to(BF16)
    return _normal(_gen(dev), dev, 1, shape.tokens, shape.hidden)


def build_layer(dev, shape: LayerShape, world: int = 1, rank: int = 0,
                process_group=None, keep_host_fp32: bool = False):
    """``RoutedDecoderLayer`` of this rank with its front end installed.  Returns
    ``(layer, front_end dict, host fp32 weights or None)``."""
    from .layer import RoutedDecoderLayer

    got = layer_weights(dev, shape, world, rank, keep_host_fp32)
    w, host = got if keep_host_fp32 else (got, None)
    (ga0, ga1), (gf0, gf1) = shape.shard(world, rank)
    hk_l = (ga1 - ga0) * (shape.kv_heads // shape.attn_groups)
    hq_l = (ga1 - ga0) * (shape.q_heads // shape.attn_groups)
    layer = RoutedDecoderLayer(w["wq"], w["wk"], w["wv"], w["wo"], w["wg"], w["wu"], w["wd"],
                               num_q_heads=hq_l, num_kv_heads=hk_l, head_dim=shape.head_dim,
                               attn_groups=ga1 - ga0, ffn_groups=gf1 - gf0, max_tokens=shape.tokens,
                               process_group=process_group)
    fe = layer_front_end(dev, shape)
    layer.set_front_end(fe["attn_router"], fe["ffn_router"], fe["n1"], fe["n2"], shape.eps,
                        (ga0, ga1) if world > 1 else None, (gf0, gf1) if world > 1 else None)
    return layer, fe, host
