"""A pruned decoder layer assembled from the routed operators (inference).

Attention block: Q, K and V projections in ONE routed ``gemm_mn`` launch over the stacked
weight ``[Wq; Wk; Wv]`` (the query channels routed by head group, the K/V channels as groups
that every token keeps), head-group-routed attention reading q, k, v as column slices of
that launch's output, routed output projection (``gemm_k``); then the dynamic-width SwiGLU
FFN.  Both sub-blocks add their input back
(residual).  Under tensor parallelism each rank holds the weights of its KV-head
groups and FFN channel groups (:mod:`dpk_b200.tp`) and the two row-parallel outputs
are summed with one all-reduce each -- the FFN router of the reference reads the
*reduced* post-attention state (``WIDE/wrapper/attn_group_ffn_block.py:197-203``), so
the two reductions cannot be merged.

This mirrors the data flow of ``WrapperDecoderLayer.forward``
(``WIDE/wrapper/attn_group_ffn_block.py:148-218``) with the routing masks given;
normalisation, rotary embedding and the routers themselves are outside this class.

With ``token_chunks > 1`` (tensor-parallel ranks, one sequence) the layer runs as a
software pipeline over chunks of query rows: projections for all tokens, then per chunk
attention + output projection, whose all-reduce runs on the collective's stream while
the next chunk's attention is computed; the FFN of a chunk starts as soon as that
chunk's first reduction has landed, and its second reduction overlaps the next chunk's
FFN.  Only the last chunk's second reduction is exposed.  A chunk of query rows
``[s,e)`` attends to keys ``[0,e)`` with the causal diagonal aligned to the bottom
right, which is exactly the causal mask of those rows in the full sequence.
"""

from __future__ import annotations

from typing import Optional

import math

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
        self.Hq, self.Hk, self.D = num_q_heads, num_kv_heads, head_dim
        self.attn_groups = attn_groups
        self.wo = wo.contiguous()
        # one stacked weight; wq / wk / wv stay available as row slices of it
        qd, kd = num_q_heads * head_dim, num_kv_heads * head_dim
        self.wqkv = torch.cat([wq, wk, wv], dim=0).contiguous()
        self.wq, self.wk, self.wv = self.wqkv[:qd], self.wqkv[qd:qd + kd], self.wqkv[qd + kd:]
        # group width of the stacked launch: divides a head group's query channels and the K/V
        # channels; 256 (one UMMA tile of output channels) where the shapes allow
        self.qkv_group = math.gcd(math.gcd(qd // attn_groups, 2 * kd), 256)
        self.fold_qkv = self.qkv_group >= 64
        self._qkv_out = None
        self._attn_out = None
        self.ffn = RoutedFFN(wg, wu, wd, ffn_groups, max_tokens)
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.timers = None          # optional dict of CUDA event pairs per phase
        self.ffn_events = None      # optional dict: event pairs around the two FFN GEMM kernels
        self.token_chunks = 1       # > 1: pipelined forward (see the module docstring)
        self.sum_o = None           # dpk_b200.peer.RowParallelSum pair: see fuse_sums()
        self.H = wo.shape[0]

    def fuse_sums(self, max_tokens: int) -> None:
        """Replace the two all-reduces by the fused row-parallel sums of
        :mod:`dpk_b200.peer`: the output and down projections store their partial sums
        into the owning ranks' memory, and the residual additions ride on the reduction.
        Collective over the process group (buffers are exchanged)."""
        from .peer import RowParallelSum
        dev, dt = self.wo.device, self.wo.dtype
        self.sum_o = RowParallelSum.connect(max_tokens, self.H, dt, dev, self.pg)
        self.ffn.row_parallel = RowParallelSum.connect(max_tokens, self.H, dt, dev, self.pg)

    def set_front_end(self, attn_router, ffn_router, input_norm_weight: torch.Tensor,
                      post_norm_weight: torch.Tensor, eps: float, attn_range=None, ffn_range=None) -> None:
        """Give the layer its own routers and norms, so that :meth:`forward_full` runs what
        ``WrapperDecoderLayer.forward`` runs (``WIDE/wrapper/attn_group_ffn_block.py:148-218``).
        ``attn_router`` / ``ffn_router``: ``(w_down [R,H], b_down, w_route [2*NG,R], b_route)`` of
        the replicated routers over ALL groups; ``attn_range`` / ``ffn_range``: the ``(g0, g1)``
        group columns this rank owns (``None`` = all)."""
        self.front = dict(attn=attn_router, ffn=ffn_router, n1=input_norm_weight.contiguous(),
                          n2=post_norm_weight.contiguous(), eps=eps, ar=attn_range, fr=ffn_range)

    def forward_full(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                     return_masks: bool = False):
        """The whole pruned layer from the residual stream ``x [B,T,H]``:

        ``execute_attn = decide(router_attention(x))``, ``h = input_layernorm(x)`` (one kernel);
        routed Q projection and dense K/V projections of ``h``; rotary embedding; routed
        attention; routed output projection, summed over the ranks, ``x1 = x + o``;
        ``execute_ffn = decide(router_ffn(x1))``, ``h2 = post_attention_layernorm(x1)`` (one
        kernel); routed FFN of ``h2``, summed over the ranks; ``x1 + y``.
        ``return_masks``: also return the two routing masks -- this rank's columns, or with
        ``return_masks="full"`` the decisions for all groups (every rank computes them)."""
        f = self.front
        B, T, H = x.shape
        self._mark("start")
        am, h, _ = ops.router_norm(x, *f["attn"], norm_weight=f["n1"], eps=f["eps"])
        am_all = am
        if f["ar"] is not None:
            am = am[..., f["ar"][0]:f["ar"][1]]
        self._mark("route1")
        q, k, v = self.project_qkv(h, am)
        ops.rope_append(q, k, None, cos, sin)
        self._mark("qkv")
        attn, meta = ops.attention_prefill(q, k, v, am, O=self._attention_out(B, T, q))
        if B != 1:
            meta = {}        # per-batch layout (attention) vs flattened layout (GEMMs)
        self._mark("attn")
        if self.sum_o is not None:
            x1 = self.sum_o.routed_gemm_k(attn.view(B, T, self.Hq * self.D), self.wo, am,
                                          residual=x.contiguous())
        else:
            if self.world > 1:
                o, _ = ops.gemm_k(attn.view(B, T, self.Hq * self.D), self.wo, am, **meta)
                dist.all_reduce(o, group=self.pg)
                x1 = x + o
            else:       # the skip connection rides on the projection's epilogue
                x1, _ = ops.gemm_k(attn.view(B, T, self.Hq * self.D), self.wo, am, residual=x, **meta)
        self._mark("oproj")
        fm, h2, _ = ops.router_norm(x1, *f["ffn"], norm_weight=f["n2"], eps=f["eps"])
        fm_all = fm
        if f["fr"] is not None:
            fm = fm[..., f["fr"][0]:f["fr"][1]]
        self._mark("route2")
        if self.ffn.row_parallel is not None:
            out = self.ffn(h2, fm, residual=x1, events=self.ffn_events)
        else:
            if self.world > 1:
                y = self.ffn(h2, fm, events=self.ffn_events)
                dist.all_reduce(y, group=self.pg)
                out = x1 + y
            else:
                out = self.ffn(h2, fm, events=self.ffn_events, residual=x1)
        self._mark("ffn")
        if return_masks == "full":
            return out, am_all, fm_all
        return (out, am, fm) if return_masks else out

    def project_qkv(self, h: torch.Tensor, attn_mask: torch.Tensor):
        """``q [B,T,Hq,D]``, ``k, v [B,T,Hk,D]`` of ``h [B,T,H]``; rows of q whose head group is
        routed out are left unwritten (attention never reads them)."""
        B, T, _ = h.shape
        qd, kd = self.Hq * self.D, self.Hk * self.D
        if not self.fold_qkv:
            q, _ = ops.gemm_mn(h, self.wq, attn_mask)
            return (q.view(B, T, self.Hq, self.D), (h @ self.wk.T).view(B, T, self.Hk, self.D),
                    (h @ self.wv.T).view(B, T, self.Hk, self.D))
        G = self.qkv_group
        per_head_group = qd // self.attn_groups // G
        m = attn_mask.reshape(B, T, self.attn_groups)
        m = m if m.dtype == torch.bool else m != 0
        stacked = torch.cat([m.repeat_interleave(per_head_group, dim=-1),
                             torch.ones((B, T, 2 * kd // G), dtype=torch.bool, device=h.device)], dim=-1)
        width = qd + 2 * kd
        if self._qkv_out is None or self._qkv_out.numel() < B * T * width or self._qkv_out.dtype != h.dtype:
            self._qkv_out = torch.empty(B * T * width, dtype=h.dtype, device=h.device)
        out = self._qkv_out[:B * T * width].view(B * T, width)
        ops.gemm_mn(h, self.wqkv, stacked, D=out)
        out = out.view(B, T, width)
        return (out[..., :qd].view(B, T, self.Hq, self.D),
                out[..., qd:qd + kd].view(B, T, self.Hk, self.D),
                out[..., qd + kd:].view(B, T, self.Hk, self.D))

    def _attention_out(self, B: int, T: int, like: torch.Tensor) -> torch.Tensor:
        """Output buffer of the attention call, allocated once and NOT zero-filled: the rows of
        routed-out (token, head group) pairs stay unwritten, and the output projection that
        reads this buffer never uses them (it clears the rows of inactive groups in shared
        memory instead of multiplying what it loaded)."""
        n = B * T * self.Hq * self.D
        if self._attn_out is None or self._attn_out.numel() < n or self._attn_out.dtype != like.dtype:
            self._attn_out = torch.empty(n, dtype=like.dtype, device=like.device)
        return self._attn_out[:n].view(B, T, self.Hq, self.D)

    def _mark(self, name):
        if self.timers is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.timers.setdefault(name, []).append(ev)

    def __call__(self, x: torch.Tensor, attn_mask: torch.Tensor, ffn_mask: torch.Tensor) -> torch.Tensor:
        """``x [B,T,H]`` (replicated), ``attn_mask [B,T,attn_groups]`` and ``ffn_mask
        [B,T,ffn_groups]`` (this rank's columns).  Returns the layer output ``[B,T,H]``."""
        B, T, H = x.shape
        if self.token_chunks > 1 and B == 1 and T >= 256 * self.token_chunks:
            if self.sum_o is not None or self.ffn.row_parallel is not None:
                raise ValueError("token_chunks > 1 pipelines NCCL all-reduces; it cannot be combined "
                                 "with fuse_sums() (the fused sums overlap by halves on their own)")
            return self._pipelined(x, attn_mask, ffn_mask)
        self._mark("start")
        q, k, v = self.project_qkv(x, attn_mask)
        self._mark("qkv")
        attn, meta = ops.attention_prefill(q, k, v, attn_mask, O=self._attention_out(B, T, q))
        if B != 1:
            meta = {}        # per-batch layout (attention) vs flattened layout (GEMMs)
        self._mark("attn")
        if self.sum_o is not None:
            # x1 = x + sum over ranks of o; layer output = x1 + sum over ranks of y
            x1 = self.sum_o.routed_gemm_k(attn.view(B, T, self.Hq * self.D), self.wo, attn_mask,
                                          residual=x.contiguous())
            self._mark("oproj")
            self._mark("ar1")
            out = self.ffn(x1, ffn_mask, residual=x1)
            self._mark("ffn")
            self._mark("ar2")
            return out
        if self.world == 1:     # both skip connections ride on the projections' epilogues
            x1, _ = ops.gemm_k(attn.view(B, T, self.Hq * self.D), self.wo, attn_mask, residual=x, **meta)
            self._mark("oproj")
            self._mark("ar1")
            out = self.ffn(x1, ffn_mask, residual=x1)
            self._mark("ffn")
            self._mark("ar2")
            return out
        o, _ = ops.gemm_k(attn.view(B, T, self.Hq * self.D), self.wo, attn_mask, **meta)
        self._mark("oproj")
        dist.all_reduce(o, group=self.pg)
        self._mark("ar1")
        x1 = x + o
        y = self.ffn(x1, ffn_mask)
        self._mark("ffn")
        dist.all_reduce(y, group=self.pg)
        self._mark("ar2")
        return x1 + y

    def _pipelined(self, x: torch.Tensor, attn_mask: torch.Tensor, ffn_mask: torch.Tensor) -> torch.Tensor:
        _, T, H = x.shape
        step = ((T + self.token_chunks - 1) // self.token_chunks + 127) // 128 * 128
        spans = [(s, min(s + step, T)) for s in range(0, T, step)]
        q, k, v = self.project_qkv(x, attn_mask)
        nopad = torch.zeros(1, dtype=torch.int32, device=x.device)     # selects bottom-right alignment
        o = torch.empty_like(x)
        y = torch.empty_like(x)
        x1 = torch.empty_like(x)
        ar1, ar2 = [], []
        if self.world == 1:
            # nothing to reduce: the skip connections ride on the projections' epilogues,
            # exactly as in the unchunked call
            for s, e in spans:
                am = attn_mask[:, s:e]
                attn, meta_c = ops.attention_prefill(q[:, s:e], k[:, :e], v[:, :e], am, Leftpad=nopad)
                ops.gemm_k(attn.view(1, e - s, self.Hq * self.D), self.wo, am, D=x1[:, s:e],
                           residual=x[:, s:e], **meta_c)
                self.ffn(x1[:, s:e], ffn_mask[:, s:e], out=y[:, s:e], residual=x1[:, s:e])
            return y
        for s, e in spans:
            am = attn_mask[:, s:e]
            attn, meta_c = ops.attention_prefill(q[:, s:e], k[:, :e], v[:, :e], am, Leftpad=nopad)
            ops.gemm_k(attn.view(1, e - s, self.Hq * self.D), self.wo, am, D=o[:, s:e], **meta_c)
            ar1.append(dist.all_reduce(o[:, s:e], group=self.pg, async_op=True))
        for (s, e), work in zip(spans, ar1):
            work.wait()                                   # the compute stream waits, not the host
            torch.add(x[:, s:e], o[:, s:e], out=x1[:, s:e])
            self.ffn(x1[:, s:e], ffn_mask[:, s:e], out=y[:, s:e])
            ar2.append(dist.all_reduce(y[:, s:e], group=self.pg, async_op=True))
        for work in ar2:
            work.wait()
        return x1.add_(y)
