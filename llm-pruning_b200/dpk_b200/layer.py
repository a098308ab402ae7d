"""A pruned decoder layer assembled from the routed operators (inference).

Attention block: routed Q projection (``gemm_mn`` over head groups), dense K/V
projections, head-group-routed attention, routed output projection (``gemm_k``);
then the dynamic-width SwiGLU FFN.  Both sub-blocks add their input back
(residual).  Under tensor parallelism each rank holds the weights of its KV-head
groups and FFN channel groups (:mod:`dpk_b200.tp`) and the two row-parallel outputs
are summed with one all-reduce each -- the FFN router of the reference reads the
*reduced* post-attention state (``WIDE/wrapper/attn_group_ffn_block.py:197-203``), so
the two reductions cannot be merged.

This mirrors the data flow of ``WrapperDecoderLayer.forward``
(``WIDE/wrapper/attn_group_ffn_block.py:148-218``) with the routing masks given;
normalisation, rotary embedding and the routers themselves are outside this class.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import ops
from .ffn import RoutedFFN


class RoutedDecoderLayer:
    def __init__(self, wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, wo: torch.Tensor,
                 wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor, *, num_q_heads: int,
                 num_kv_heads: int, head_dim: int, attn_groups: int, ffn_groups: int,
                 max_tokens: int, process_group: Optional[dist.ProcessGroup] = None):
        """All weights are this rank's slices: ``wq [Hq_l*D, H]``, ``wk/wv [Hk_l*D, H]``,
        ``wo [H, Hq_l*D]``, ``wg/wu [I_l, H]``, ``wd [H, I_l]``; the head and group counts
        are local too."""
        self.wq, self.wk, self.wv, self.wo = (w.contiguous() for w in (wq, wk, wv, wo))
        self.Hq, self.Hk, self.D = num_q_heads, num_kv_heads, head_dim
        self.attn_groups = attn_groups
        self.ffn = RoutedFFN(wg, wu, wd, ffn_groups, max_tokens)
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.timers = None          # optional dict of CUDA event pairs per phase

    def _mark(self, name):
        if self.timers is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.timers.setdefault(name, []).append(ev)

    def __call__(self, x: torch.Tensor, attn_mask: torch.Tensor, ffn_mask: torch.Tensor) -> torch.Tensor:
        """``x [B,T,H]`` (replicated), ``attn_mask [B,T,attn_groups]`` and ``ffn_mask
        [B,T,ffn_groups]`` (this rank's columns).  Returns the layer output ``[B,T,H]``."""
        B, T, H = x.shape
        self._mark("start")
        q, meta = ops.gemm_mn(x, self.wq, attn_mask)
        k = (x @ self.wk.T).view(B, T, self.Hk, self.D)
        v = (x @ self.wv.T).view(B, T, self.Hk, self.D)
        self._mark("qkv")
        meta_attn = meta if B == 1 else {}       # per-batch vs flattened layouts differ for B > 1
        attn, _ = ops.attention_prefill(q.view(B, T, self.Hq, self.D), k, v, attn_mask, **meta_attn)
        self._mark("attn")
        o, _ = ops.gemm_k(attn.view(B, T, self.Hq * self.D), self.wo, attn_mask, **meta)
        self._mark("oproj")
        if self.world > 1:
            dist.all_reduce(o, group=self.pg)
        self._mark("ar1")
        x1 = x + o
        y = self.ffn(x1, ffn_mask)
        self._mark("ffn")
        if self.world > 1:
            dist.all_reduce(y, group=self.pg)
        self._mark("ar2")
        return x1 + y
