"""Drop-in bodies for the model-wrapper call sites that consume the routed operators.

The reference's wrappers compute densely and multiply by the routing mask so that
training stays differentiable:

* ``WrapperMLP.forward`` -- ``down_proj(apply_mask(swiglu(gate_proj(x), up_proj(x)),
  execute_ffn))`` (``WIDE/wrapper/attn_group_ffn_block.py:28-39``, ``apply_mask`` in
  ``WIDE/wrapper/base_layer.py:42-70``);
* ``WrapperAttention.forward`` -- FlashAttention-2 followed by ``attn_output *
  head_mask`` and ``o_proj`` (``attn_group_ffn_block.py:73-97``);
* LFF's block -- ``self.block.mlp(x) * gate`` / ``self.block.self_attn(x) * gate`` with a
  per-token gate (``LFF/router_attn_mlp.py:405-430, 461-476``).

At inference the masks are hard 0/1 tensors in the activation dtype
(``base_layer.py:204-207``), so the same results come from kernels that skip the
routed-out work.  The classes below keep the wrappers' argument names; tensors use
the wrappers' sequence-first layouts (``[B,S,H]`` hidden states, ``[B,S,heads,D]``
q/k/v, which is also the layout of ``WIDE/wrapper/cache.py:10-46``).
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import ops
from .ffn import RoutedFFN


def as_bool_mask(execute: Optional[torch.Tensor], batch: int, seq: int, groups: int,
                 device) -> torch.Tensor:
    """0/1 routing tensor of any dtype (or ``None`` = keep everything) -> bool
    ``[B,S,groups]``; a ``[B,S]`` tensor is one group per token."""
    if execute is None:
        return torch.ones((batch, seq, groups), dtype=torch.bool, device=device)
    if execute.dim() == 2:
        execute = execute[..., None]
    if execute.shape != (batch, seq, groups):
        raise ValueError(f"Mask has shape {tuple(execute.shape)}, expected {(batch, seq, groups)}")
    return execute != 0


class RoutedMLP(nn.Module):
    """Body of ``WrapperMLP.forward(hidden_states, execute_ffn)`` on the routed kernels.

    ``gate_proj``, ``up_proj``, ``down_proj`` are the block's bias-free ``nn.Linear``
    modules; ``ffn_group_size`` is the wrapper's group width (128 in the reference's
    configurations).  ``max_tokens`` bounds ``B*S`` of a call (workspace size).
    """

    def __init__(self, gate_proj: nn.Linear, up_proj: nn.Linear, down_proj: nn.Linear,
                 ffn_group_size: int, max_tokens: int):
        super().__init__()
        for lin in (gate_proj, up_proj, down_proj):
            if lin.bias is not None:
                raise ValueError("the routed FFN kernels take bias-free projections")
        inter = gate_proj.weight.shape[0]
        if inter % ffn_group_size:
            raise ValueError(f"group_size={ffn_group_size} must divide feature size {inter}")
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj
        self.ffn_group_size = ffn_group_size
        self.group_num = inter // ffn_group_size
        self.max_tokens = max_tokens
        self._plan: Optional[RoutedFFN] = None

    def _ffn(self) -> RoutedFFN:
        if self._plan is None:
            self._plan = RoutedFFN(self.gate_proj.weight.detach(), self.up_proj.weight.detach(),
                                   self.down_proj.weight.detach(), self.group_num, self.max_tokens)
        return self._plan

    def forward(self, hidden_states: torch.Tensor,
                execute_ffn: Optional[torch.Tensor] = None) -> torch.Tensor:
        b, s, _ = hidden_states.shape
        mask = as_bool_mask(execute_ffn, b, s, self.group_num, hidden_states.device)
        return self._ffn()(hidden_states, mask)


def token_gated_mlp(mlp: RoutedMLP, hidden_states: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """LFF's ``self.block.mlp(x) * gate[..., None]`` for a hard per-token gate
    (``LFF/router_attn_mlp.py:461-476``): tokens whose gate is 0 are not computed."""
    b, s, _ = hidden_states.shape
    keep = (gate != 0)[..., None].expand(b, s, mlp.group_num)
    return mlp(hidden_states, keep)


def routed_attention(query_states: torch.Tensor, key_states: torch.Tensor,
                     value_states: torch.Tensor, execute_attn: Optional[torch.Tensor],
                     scaling: Optional[float] = None, is_causal: bool = True) -> torch.Tensor:
    """The attention core of ``WrapperAttention.forward``: FlashAttention followed by
    ``attn_output * head_mask`` (``attn_group_ffn_block.py:73-94``), computed only for
    the routed-in (token, head group) pairs.

    ``query_states [B,S,Hq,D]``; ``key_states/value_states [B,T,Hk,D]`` (the cache's
    layout); ``execute_attn [B,S,Hq/attn_group_size]`` 0/1.  Returns ``[B,S,Hq,D]``.
    One query token per sequence takes the split-KV decode kernel.
    """
    b, s, hq, _ = query_states.shape
    if execute_attn is None:
        groups = key_states.shape[2]          # every KV-head group stays active
    elif execute_attn.dim() == 2:
        groups = 1                            # token-level routing
    else:
        groups = execute_attn.shape[-1]
    mask = as_bool_mask(execute_attn, b, s, groups, query_states.device)
    if s == 1:
        out, _ = ops.attention_decode(query_states, key_states, value_states, mask, scale=scaling)
    else:
        out, _ = ops.attention_prefill(query_states, key_states, value_states, mask, scale=scaling,
                                       is_causal=is_causal)
    return out


def routed_q_proj(hidden_states: torch.Tensor, q_weight: torch.Tensor,
                  execute_attn: torch.Tensor, metadata: Optional[dict] = None):
    """``q_proj`` restricted to the routed-in head groups: a ``gemm_mn`` whose groups are
    ``attn_group_size * head_dim`` output channels wide.  Returns ``(q, metadata)``;
    the metadata can be passed on to :func:`routed_o_proj` (the reference's tested
    metadata reuse, ``DynamicPruningKernels/tests/test_gpu_smoke.py:256-292``)."""
    b, s, _ = hidden_states.shape
    mask = as_bool_mask(execute_attn, b, s, execute_attn.shape[-1], hidden_states.device)
    return ops.gemm_mn(hidden_states, q_weight, mask, **(metadata or {}))


def routed_o_proj(attn_output: torch.Tensor, o_weight: torch.Tensor, execute_attn: torch.Tensor,
                  metadata: Optional[dict] = None):
    """``o_proj(attn_output.flatten(-2))`` skipping the routed-out head groups: a
    ``gemm_k`` over ``Hq*D`` inputs in ``NG`` groups (``attn_group_ffn_block.py:96-97``)."""
    b, s = attn_output.shape[:2]
    flat = attn_output.reshape(b, s, -1)
    mask = as_bool_mask(execute_attn, b, s, execute_attn.shape[-1], attn_output.device)
    return ops.gemm_k(flat, o_weight, mask, **(metadata or {}))


class RoutedTokenRouter(nn.Module):
    """``TokenRouter`` (``WIDE/wrapper/base_layer.py:89-114``) with the evaluation-time decision
    of ``WrapperDecoderLayer._gumbel_softmax`` (``:204-207``) computed by one kernel.

    Parameter names follow the reference module (``compressor``, ``router``), so its state dict
    loads unchanged.  ``decide`` returns what the layer derives from the router at inference --
    ``execute`` / ``skip`` as 0/1 tensors in the activation dtype, ``[B,S,group_num]`` -- and,
    when the layer norm that reads the same hidden state is passed, its output as well
    (``WIDE/wrapper/attn_group_ffn_block.py:170-176``: ``input_layernorm(hidden_states)`` next
    to ``router_attention(residual)``)."""

    def __init__(self, hidden_size: int, group_num: int, rank_size: int = 16):
        super().__init__()
        if group_num <= 0 or not 0 < rank_size <= 16:
            raise ValueError("group_num must be positive and rank_size in 1..16")
        self.compressor = nn.Linear(hidden_size, rank_size)
        self.router = nn.Linear(rank_size, group_num * 2)
        self.group_num = group_num

    def decide(self, hidden_states: torch.Tensor, norm: Optional[nn.Module] = None):
        """``norm``: an RMSNorm module with ``weight`` and ``variance_epsilon`` (or ``eps``)."""
        weight = eps = None
        if norm is not None:
            weight = norm.weight
            eps = getattr(norm, "variance_epsilon", getattr(norm, "eps", 1e-6))
        execute, normed, _ = ops.router_norm(
            hidden_states, self.compressor.weight, self.compressor.bias, self.router.weight,
            self.router.bias, norm_weight=weight, eps=eps if eps is not None else 1e-6)
        dt = hidden_states.dtype
        return execute.to(dt), execute.logical_not().to(dt), normed


class SeqFirstKVCache:
    """Preallocated counterpart of ``DynamicLayerSeqFirstLayer`` (``WIDE/wrapper/cache.py:10-60``):
    keys and values stay ``[B,T,Hk,D]`` but live in one ``[B,capacity,Hk,D]`` allocation per
    tensor, and ``rope_update`` applies the rotary embedding and writes the new rows in place
    (the reference rotates first and then concatenates, ``attn_group_ffn_block.py:60-67``)."""

    def __init__(self, batch: int, capacity: int, num_kv_heads: int, head_dim: int,
                 dtype: torch.dtype, device):
        shape = (batch, capacity, num_kv_heads, head_dim)
        self.keys = torch.empty(shape, dtype=dtype, device=device)
        self.values = torch.empty(shape, dtype=dtype, device=device)
        self.length = 0

    def get_seq_length(self) -> int:
        return self.length

    def rope_update(self, query_states: torch.Tensor, key_states: torch.Tensor,
                    value_states: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
        """Returns ``(rotated queries, keys[:, :length], values[:, :length])``."""
        q, keys, values = ops.rope_append(query_states, key_states, value_states, cos, sin,
                                          self.keys, self.values, self.length)
        self.length += key_states.shape[1]
        return q, keys, values
