"""The MLP kernel call convention of the reference's inference simulator on the routed kernels.

``PruningInferSim`` looks its MLP kernels up by name and calls ``Kernel.base_prefill(x=..., w_up=...,
w_gate=..., w_down=..., b_up=..., b_gate=..., route_mask=..., activation=..., estimated_sparsity=...,
impl=..., backend=...)`` (``PruningInferSim/ops/mlp/m_pruning.py:39-105``; registry of kernels
``PruningInferSim/ops/__init__.py:78-82``).  ``RoutedMLPKernel`` takes the same keywords:

* ``w_gate`` and ``w_down`` given: the SwiGLU-style block ``down(act(gate(x)) * up(x))`` restricted to
  the routed tokens / groups -- one call of :func:`dpk_b200.ops.ffn_swiglu` when the activation is
  SiLU and there are no biases, else the same composition from ``gemm_mn`` and ``gemm_k``;
* only ``w_up``: a single routed linear layer (``gemm_mn``).

``route_mask`` is ``[B,S]`` (the simulator's token-wise pruning: a token keeps or skips the whole
layer) or ``[B,S,NG]`` (channel groups).  ``estimated_sparsity``, ``impl`` and ``backend`` are
accepted for call compatibility; there is one implementation here.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import ops


def _mask3(route_mask: Optional[torch.Tensor], x: torch.Tensor) -> torch.Tensor:
    b, s, _ = x.shape
    if route_mask is None:
        return torch.ones((b, s, 1), dtype=torch.bool, device=x.device)
    m = route_mask if route_mask.dim() == 3 else route_mask[..., None]
    if m.shape[:2] != (b, s):
        raise ValueError(f"route_mask has shape {tuple(route_mask.shape)}, expected [{b},{s}] or [{b},{s},NG]")
    return m != 0


def _add_bias(y: torch.Tensor, bias: Optional[torch.Tensor], mask: torch.Tensor) -> torch.Tensor:
    """Bias of a routed output-width projection: only where the (token, group) block is active."""
    if bias is None:
        return y
    groups = mask.shape[-1]
    on = mask.repeat_interleave(y.shape[-1] // groups, dim=-1)
    return y + bias.to(y.dtype) * on.to(y.dtype)


class RoutedMLPKernel:
    @classmethod
    def base_prefill(cls, x: torch.Tensor, w_up: torch.Tensor, w_gate: Optional[torch.Tensor] = None,
                     w_down: Optional[torch.Tensor] = None, b_up: Optional[torch.Tensor] = None,
                     b_gate: Optional[torch.Tensor] = None, route_mask: Optional[torch.Tensor] = None,
                     activation: Optional[str] = "identity", estimated_sparsity: Optional[float] = 0,
                     impl: Optional[str] = "auto", **kwargs) -> torch.Tensor:
        mask = _mask3(route_mask, x)
        if w_down is None and w_gate is None:                 # a single routed linear layer
            y, _ = ops.gemm_mn(x, w_up, mask, activation=activation or "identity")
            if b_up is not None:
                if (activation or "identity") != "identity":
                    raise ValueError("a bias in front of the activation is not fused: pass activation='identity'")
                y = _add_bias(y, b_up, mask)
            return y
        if w_gate is None or w_down is None:
            raise ValueError("w_gate and w_down go together")
        if (activation or "identity") == "silu" and b_up is None and b_gate is None:
            return ops.ffn_swiglu(x, w_gate, w_up, w_down, mask)
        up, meta = ops.gemm_mn(x, w_up, mask)
        up = _add_bias(up, b_up, mask)
        if b_gate is None:
            gate, _ = ops.gemm_mn(x, w_gate, mask, activation=activation or "identity", **meta)
        else:
            gate, _ = ops.gemm_mn(x, w_gate, mask, **meta)
            gate = _add_bias(gate, b_gate, mask)
            act = {"identity": lambda t: t, "relu": torch.relu, "silu": torch.nn.functional.silu}
            on = mask.repeat_interleave(gate.shape[-1] // mask.shape[-1], dim=-1)
            gate = act[activation or "identity"](gate) * on.to(gate.dtype)
        out, _ = ops.gemm_k(gate * up, w_down, mask, **meta)
        return out

    @classmethod
    def base_decode(cls, **kwargs) -> torch.Tensor:
        return cls.base_prefill(**kwargs)
