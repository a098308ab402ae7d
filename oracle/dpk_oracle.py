"""CPU oracle for the routed dynamic-width operators.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain fp32 PyTorch on the CPU, what the reference's
PyTorch backend computes for the four operator families and for the routing
layout that precedes them.  It exists so that the CUDA kernels can be checked
against an independent statement of the semantics.  Nothing in the shipped
package imports it; only the tests, the smoke entry and the CPU-baseline leg of
the benchmark do.

Parity status: PINNED.  ``tests/golden/*.npz`` were produced by running the
reference's own ``run_kernel(..., backend="torch")`` on seeded inputs (see
``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` checks every
function below against them, including the reference's hand-written
known-answer cases (``DynamicPruningKernels/tests/test_references.py:11-84``).

Each function cites the reference lines it follows.  The formulations are
deliberately different from the reference's (explicit per-group loops and an
explicit softmax instead of dense-then-mask and SDPA) so that an error in one
is unlikely to be mirrored in the other.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

__all__ = [
    "as_group_mask",
    "topk_route_mask",
    "route_compact",
    "bottleneck_router",
    "rms_norm",
    "rope",
    "kv_append",
    "gemm_mn",
    "gemm_k",
    "ffn_swiglu",
    "attention",
    "attention_prefill",
    "attention_decode",
    "dense_then_mask_ffn",
    "decoder_layer_rows",
    "dense_then_mask_layer_rows",
    "rel_err",
    "rel_err_active",
    "rel_err_rows",
]


# ----------------------------------------------------------------------------
# routing
# ----------------------------------------------------------------------------

def as_group_mask(mask: torch.Tensor, batch: int, tokens: int) -> torch.Tensor:
    """``[B,T]`` or ``[B,T,NG]`` of any dtype -> bool ``[B,T,NG]``.

    Follows ``DynamicPruningKernels/python/references.py:11-19``: a 2-D mask is
    one group spanning the whole width (whole-token skip).
    """
    if mask.dim() == 2:
        mask = mask[..., None]
    if mask.dim() != 3 or tuple(mask.shape[:2]) != (batch, tokens):
        raise ValueError("Mask must have shape [batch, tokens] or [batch, tokens, groups]")
    return mask != 0


def topk_route_mask(logits: torch.Tensor, keep: int) -> torch.Tensor:
    """Benchmark-defined router: each token keeps its ``keep`` largest logits.

    The reference ships no top-k router (its kernels take a ready Boolean
    mask, ``DynamicPruningKernels/README.md:35``; WIDE's evaluation routing is
    a 2-way argmax, ``WIDE/wrapper/base_layer.py:204-207``).  Ties are broken
    towards the lower group index, which is what the CUDA router does.
    """
    if not 0 <= keep <= logits.shape[-1]:
        raise ValueError("keep out of range")
    l32 = logits.to(torch.float32)
    order = torch.sort(l32, dim=-1, descending=True, stable=True).indices
    mask = torch.zeros(l32.shape, dtype=torch.bool)
    mask.scatter_(-1, order[..., :keep], True)
    return mask


def _round_to(t: torch.Tensor, dtype: Optional[torch.dtype]) -> torch.Tensor:
    return t if dtype is None else t.to(dtype).to(torch.float32)


def bottleneck_router(x: torch.Tensor, w_down: torch.Tensor, b_down: Optional[torch.Tensor],
                      w_route: torch.Tensor, b_route: Optional[torch.Tensor],
                      module_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Two-stage token router and its evaluation-time decision.

    ``logits = (x @ w_down.T + b_down) @ w_route.T + b_route`` reshaped to ``[..., NG, 2]``
    (``WIDE/wrapper/base_layer.py:89-114`` ``TokenRouter``; the same arithmetic as
    ``PruningInferSim/ops/router.py:85-126`` ``BottleneckRouter``).  A group is executed
    when the argmax over the pair is index 0 -- ``skip = argmax(-1).bool(); execute = ~skip``
    (``base_layer.py:204-207``) -- and ``argmax`` returns the first index on a tie, so
    ``execute = logits[..., 0] >= logits[..., 1]``.

    ``module_dtype`` (bf16 / fp16) reproduces the rounding of a module that runs in that
    dtype: the output of each ``nn.Linear`` is rounded once (fp32 accumulation, bias added
    before the rounding).  ``None`` keeps everything in fp32.
    Returns ``(logits float32 [..., NG, 2], execute bool [..., NG])``.
    """
    xf = x.to(torch.float32)
    c = xf @ w_down.to(torch.float32).T
    if b_down is not None:
        c = c + b_down.to(torch.float32)
    c = _round_to(c, module_dtype)
    l = c @ w_route.to(torch.float32).T
    if b_route is not None:
        l = l + b_route.to(torch.float32)
    l = _round_to(l, module_dtype)
    if l.shape[-1] % 2:
        raise ValueError("the router must produce two logits per group")
    l = l.reshape(*l.shape[:-1], l.shape[-1] // 2, 2)
    return l, l[..., 0] >= l[..., 1]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm as the wrapped decoder layers apply it (``input_layernorm`` /
    ``post_attention_layernorm``, ``WIDE/wrapper/attn_group_ffn_block.py:170,195``; the
    modules are the Hugging Face ``LlamaRMSNorm`` of transformers 5.5, a third-party
    dependency of the reference): statistics in fp32, the normalised value rounded to the
    input dtype, then multiplied by the weight in that dtype."""
    dt = x.dtype
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    y = (xf * torch.rsqrt(var + eps)).to(dt)
    return weight.to(dt) * y


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of ``x [B,T,heads,D]`` with ``cos, sin [B or 1, T, D]``:
    ``x*cos + rotate_half(x)*sin`` with ``rotate_half(x) = cat(-x[..., D/2:], x[..., :D/2])``
    (``WIDE/wrapper/base_layer.py:18-44``), written per half instead of through the
    concatenation.  fp32 arithmetic; the caller rounds."""
    xf, c, s_ = x.to(torch.float32), cos.to(torch.float32)[:, :, None, :], sin.to(torch.float32)[:, :, None, :]
    half = x.shape[-1] // 2
    lo, hi = xf[..., :half], xf[..., half:]
    out = torch.empty_like(xf)
    out[..., :half] = lo * c[..., :half] - hi * s_[..., :half]
    out[..., half:] = hi * c[..., half:] + lo * s_[..., half:]
    return out


def kv_append(k_cache: torch.Tensor, v_cache: torch.Tensor, past_len: int, k: torch.Tensor,
              v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sequence-first KV cache update: the reference layer returns ``cat([keys, k], dim=1)``
    and the same for the values (``WIDE/wrapper/cache.py:24-46``); with a preallocated
    ``[B,capacity,Hk,D]`` cache that is a write of rows ``past_len .. past_len+T-1`` and a view
    of the first ``past_len+T`` rows."""
    T = k.shape[1]
    if past_len + T > k_cache.shape[1]:
        raise ValueError("cache capacity exceeded")
    k_cache[:, past_len:past_len + T] = k
    v_cache[:, past_len:past_len + T] = v
    return k_cache[:, :past_len + T], v_cache[:, :past_len + T]


def route_compact(mask2d: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Routing layout for a flattened ``[M,NG]`` mask.

    Returns ``(sorted_mask bool[M,NG], sorted_indices int64[M,NG], counts
    int32[NG])``: per group column the active rows first, in ascending row
    order, then the inactive rows in ascending order.  The reference builds
    the same layout with ``torch.sort(mask, dim=0, descending=True,
    stable=False)`` (``python/gemm_mn/jit.py:410-415``); its kernels rely only
    on "all True rows precede all False rows" (``include/gemm_mn/v1/sm12x.cuh:
    272-311``).  The order among equal keys is unspecified there; this build
    fixes the stable order, so this oracle is a plain loop.
    """
    m = (mask2d != 0)
    M, NG = m.shape
    smask = torch.zeros((M, NG), dtype=torch.bool)
    sidx = torch.zeros((M, NG), dtype=torch.int64)
    counts = torch.zeros((NG,), dtype=torch.int32)
    rows = torch.arange(M, dtype=torch.int64)
    for g in range(NG):
        col = m[:, g]
        act = rows[col]
        ina = rows[~col]
        c = act.numel()
        counts[g] = c
        smask[:c, g] = True
        sidx[:c, g] = act
        sidx[c:, g] = ina
    return smask, sidx, counts


# ----------------------------------------------------------------------------
# routed GEMMs
# ----------------------------------------------------------------------------

def _act(x: torch.Tensor, activation: str) -> torch.Tensor:
    if activation == "identity":
        return x
    if activation == "relu":
        return torch.clamp_min(x, 0)
    if activation == "silu":
        return x / (1.0 + torch.exp(-x))
    raise ValueError(f"Unsupported activation: {activation}")


def gemm_mn(A: torch.Tensor, W: torch.Tensor, mask: torch.Tensor,
            activation: str = "identity") -> torch.Tensor:
    """Output-width routed projection.

    ``D[b,t, g*G:(g+1)*G] = act(A[b,t,:] @ W[g*G:(g+1)*G,:]^T)`` where group
    ``g`` is active for token ``(b,t)``, zero elsewhere
    (``python/references.py:29-61``; act(0)=0 for all three activations so
    masking before or after the activation is the same).
    """
    if A.dim() != 3 or W.dim() != 2:
        raise ValueError("A must be [B, T, K] and W must be [N, K]")
    B, T, K = A.shape
    N = W.shape[0]
    gm = as_group_mask(mask, B, T)
    NG = gm.shape[-1]
    if N % NG:
        raise ValueError(f"Output width {N} must be divisible by groups {NG}")
    G = N // NG
    a = A.reshape(B * T, K).to(torch.float32)
    w = W.to(torch.float32)
    gm2 = gm.reshape(B * T, NG)
    out = torch.zeros((B * T, N), dtype=torch.float32)
    for g in range(NG):
        rows = torch.nonzero(gm2[:, g]).flatten()
        if rows.numel() == 0:
            continue
        out[rows, g * G:(g + 1) * G] = _act(a[rows] @ w[g * G:(g + 1) * G].T, activation)
    return out.reshape(B, T, N)


def gemm_k(A: torch.Tensor, W: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Reduction-width routed projection.

    ``D[b,t,:] = sum over active g of A[b,t, g*G:(g+1)*G] @ W[:, g*G:(g+1)*G]^T``
    (``python/references.py:64-86``).  Whatever the caller left in the
    inactive column blocks of ``A`` does not contribute.
    """
    if A.dim() != 3 or W.dim() != 2:
        raise ValueError("A must be [B, T, K] and W must be [N, K]")
    B, T, K = A.shape
    N = W.shape[0]
    gm = as_group_mask(mask, B, T)
    NG = gm.shape[-1]
    if K % NG:
        raise ValueError(f"Input width {K} must be divisible by groups {NG}")
    G = K // NG
    a = A.reshape(B * T, K).to(torch.float32)
    w = W.to(torch.float32)
    gm2 = gm.reshape(B * T, NG)
    out = torch.zeros((B * T, N), dtype=torch.float32)
    for g in range(NG):
        rows = torch.nonzero(gm2[:, g]).flatten()
        if rows.numel() == 0:
            continue
        out[rows] += a[rows, g * G:(g + 1) * G] @ w[:, g * G:(g + 1) * G].T
    return out.reshape(B, T, N)


def ffn_swiglu(x: torch.Tensor, Wg: torch.Tensor, Wu: torch.Tensor, Wd: torch.Tensor,
               mask: torch.Tensor, round_intermediate: Optional[torch.dtype] = None) -> torch.Tensor:
    """Dynamic-width SwiGLU FFN: ``down(mask * silu(gate(x)) * up(x))``.

    Composition used by the reference's callers:
    ``gemm_k(gemm_mn(x,Wg,silu) * gemm_mn(x,Wu), Wd)``
    (``PruningInferSim/ops/mlp/m_pruning.py:76-105``), equal to WIDE's
    ``down_proj(apply_mask(swiglu(gate_proj(x), up_proj(x))))``
    (``WIDE/wrapper/attn_group_ffn_block.py:33-38``).  ``round_intermediate``
    optionally rounds the intermediate to the GPU's storage dtype so that the
    comparison isolates kernel error from the unavoidable bf16 hand-off.
    """
    h = gemm_mn(x, Wg, mask, "silu") * gemm_mn(x, Wu, mask, "identity")
    if round_intermediate is not None:
        h = h.to(round_intermediate).to(torch.float32)
    return gemm_k(h, Wd, mask)


def dense_then_mask_ffn(x, Wg, Wu, Wd, mask):
    """The reference CPU path's cost model: dense GEMMs, then mask.

    ``python/references.py:50-53, 83-85`` compute the full-width product and
    ``masked_fill`` afterwards, so on the CPU the routed FFN costs as much as
    the dense one.  Used only as the timed CPU baseline.
    """
    B, T, _ = x.shape
    gm = as_group_mask(mask, B, T)
    NG = gm.shape[-1]
    x32, wg, wu, wd = (t.to(torch.float32) for t in (x, Wg, Wu, Wd))
    gate = torch.nn.functional.silu(x32 @ wg.T)
    up = x32 @ wu.T
    h = (gate * up).reshape(B, T, NG, -1)
    h = h.masked_fill(~gm[..., None], 0).reshape(B, T, -1)
    return h @ wd.T


# ----------------------------------------------------------------------------
# routed attention
# ----------------------------------------------------------------------------

def attention(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, mask: torch.Tensor,
              scale: Optional[float] = None, leftpad: Optional[torch.Tensor] = None,
              is_causal: bool = False, q_chunk: int = 1024,
              q_positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Query-head-group routed attention (``python/references.py:89-149``).

    ``Q,O: [B,Tq,Hq,D]``; ``K,V: [B,Tk,Hk,D]``; ``mask: [B,Tq,NG]``.  Group
    ``g`` is the ``Hq/NG`` consecutive query heads ``[g*Hq/NG, (g+1)*Hq/NG)``;
    query head ``h`` reads KV head ``h // (Hq/Hk)``.  Inactive (token, group)
    pairs give zero output rows.  Causal alignment follows the reference's
    PyTorch path exactly: top-left (``k <= q``, SDPA's ``is_causal``) when no
    ``Leftpad`` is given, bottom-right (``k <= q + Tk - Tq``) when one is
    (``references.py:123-139``); the two agree when ``Tq == Tk``.  Keys
    ``k < leftpad[b]`` are excluded.

    ``q_positions`` (int64 ``[Tq]``): the sequence position of each query row when ``Q`` holds
    a sample of the rows of a longer sequence (rows of attention are independent, so a
    full-size case can be checked on a sample); causal masking then uses these positions.
    """
    if Q.dim() != 4 or K.dim() != 4 or V.dim() != 4:
        raise ValueError("Q, K, and V must have shape [B, T, H, D]")
    if K.shape != V.shape:
        raise ValueError("K and V must have matching shapes")
    B, Tq, Hq, D = Q.shape
    Tk, Hk = K.shape[1], K.shape[2]
    gm = as_group_mask(mask, B, Tq)
    NG = gm.shape[-1]
    if Hq % NG:
        raise ValueError(f"Query heads {Hq} must be divisible by groups {NG}")
    if Hq % Hk:
        raise ValueError("Hq must be a multiple of Hk")
    hpg = Hq // NG
    rep = Hq // Hk
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros((B, Tq, Hq, D), dtype=torch.float32)
    kpos = torch.arange(Tk)
    causal_shift = (Tk - Tq) if leftpad is not None else 0
    if q_positions is not None:
        if leftpad is not None or q_positions.shape != (Tq,):
            raise ValueError("q_positions is a [Tq] vector and excludes Leftpad")
        qpos = q_positions.to(torch.int64)
    else:
        qpos = torch.arange(Tq)
    for b in range(B):
        lp = int(leftpad[b]) if leftpad is not None else 0
        for h in range(Hq):
            g = h // hpg
            rows = torch.nonzero(gm[b, :, g]).flatten()
            if rows.numel() == 0:
                continue
            kh = K[b, :, h // rep, :].to(torch.float32)
            vh = V[b, :, h // rep, :].to(torch.float32)
            for c0 in range(0, rows.numel(), q_chunk):
                r = rows[c0:c0 + q_chunk]
                q = Q[b, r, h, :].to(torch.float32)
                s = (q @ kh.T) * sc
                allow = (kpos[None, :] >= lp)
                if is_causal:
                    allow = allow & (kpos[None, :] <= (qpos[r][:, None] + causal_shift))
                s = s.masked_fill(~allow, float("-inf"))
                mx = s.max(dim=-1, keepdim=True).values
                mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
                p = torch.exp(s - mx)
                den = p.sum(dim=-1, keepdim=True)
                # a row with every key excluded (query before its batch's leftpad
                # under causal masking) comes out as zeros from the reference's
                # SDPA call; keep that
                o = torch.where(den > 0, (p @ vh) / den, torch.zeros(()))
                out[b, r, h, :] = o
    return out


def attention_prefill(Q, K, V, mask, **kw):
    """``python/references.py:152-163``: causal unless told otherwise."""
    kw.setdefault("is_causal", True)
    return attention(Q, K, V, mask, **kw)


def attention_decode(Q, K, V, mask, **kw):
    """``python/references.py:166-175``: one query token, non-causal."""
    kw.setdefault("is_causal", False)
    return attention(Q, K, V, mask, **kw)


# ----------------------------------------------------------------------------
# the pruned decoder layer on a sample of its token rows
# ----------------------------------------------------------------------------

def decoder_layer_rows(x: torch.Tensor, rows: torch.Tensor, w: dict, attn_mask_rows: torch.Tensor,
                       ffn_mask_rows: torch.Tensor, *, num_q_heads: int, num_kv_heads: int,
                       head_dim: int, norm1: Optional[torch.Tensor] = None,
                       norm2: Optional[torch.Tensor] = None, eps: float = 1e-5,
                       cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                       handoff: Optional[torch.dtype] = None, return_x1: bool = False):
    """Output rows ``rows`` of the pruned decoder layer for one sequence ``x [1,T,H]``.

    Data flow of ``WrapperDecoderLayer.forward`` (``WIDE/wrapper/attn_group_ffn_block.py:
    148-218``) with the routing decisions given: ``h = input_layernorm(x)``; routed Q
    projection, dense K/V projections, rotary embedding, head-group-routed causal
    attention, routed output projection, ``x1 = x + o``; ``h2 = post_attention_layernorm(x1)``;
    routed SwiGLU FFN; ``x1 + y``.  Every step after the K/V projections is independent per
    token, so only the sampled rows are computed; K and V are computed for all tokens.

    ``w``: fp32 ``wq [Hq*D,H]``, ``wk, wv [Hk*D,H]``, ``wo [H,Hq*D]``, ``wg, wu [I,H]``,
    ``wd [H,I]``.  ``attn_mask_rows [1,R,NGa]`` / ``ffn_mask_rows [1,R,NGf]``: the decisions
    for the sampled rows.  ``norm1/norm2`` ``None`` = no normalisation, ``cos/sin [T,D]``
    ``None`` = no rotary embedding.  ``handoff`` (e.g. bf16) rounds every tensor that the GPU
    path stores in that dtype between two kernels; ``None`` keeps fp32 throughout.
    """
    if x.dim() != 3 or x.shape[0] != 1:
        raise ValueError("x must be [1,T,H]")
    T, H = x.shape[1], x.shape[2]
    Hq, Hk, D = num_q_heads, num_kv_heads, head_dim
    rows = rows.to(torch.int64)
    R = rows.numel()
    rd = (lambda t: _round_to(t, handoff))
    xf = x.to(torch.float32)
    if norm1 is not None:
        h = rms_norm(xf if handoff is None else xf.to(handoff), norm1, eps).to(torch.float32)
    else:
        h = xf
    k = rd(h[0] @ w["wk"].T).view(1, T, Hk, D)
    v = rd(h[0] @ w["wv"].T).view(1, T, Hk, D)
    hr = h[:, rows]
    q = rd(gemm_mn(hr, w["wq"], attn_mask_rows)).view(1, R, Hq, D)
    if cos is not None:
        c32, s32 = cos.to(torch.float32)[None], sin.to(torch.float32)[None]
        k = rd(rope(k, c32, s32))
        q = rd(rope(q, c32[:, rows], s32[:, rows]))
    a = rd(attention(q, k, v, attn_mask_rows, is_causal=True, q_positions=rows)).view(1, R, Hq * D)
    x1 = rd(xf[:, rows] + rd(gemm_k(a, w["wo"], attn_mask_rows)))
    if norm2 is not None:
        h2 = rms_norm(x1 if handoff is None else x1.to(handoff), norm2, eps).to(torch.float32)
    else:
        h2 = x1
    y = ffn_swiglu(h2, w["wg"], w["wu"], w["wd"], ffn_mask_rows, round_intermediate=handoff)
    out = x1 + y
    return (out, x1) if return_x1 else out


def dense_then_mask_layer_rows(x: torch.Tensor, rows: torch.Tensor, w: dict, k: torch.Tensor,
                               v: torch.Tensor, attn_mask_rows: torch.Tensor,
                               ffn_mask_rows: torch.Tensor, *, num_q_heads: int, num_kv_heads: int,
                               head_dim: int) -> torch.Tensor:
    """Cost model of the reference's CPU path for the same layer, on a sample of token rows:
    every operator computes the dense product (or dense attention over all heads, SDPA as in
    ``python/references.py:131-139``) and masks afterwards (``references.py:50-53, 83-85,
    141-148``).  The K/V projections are computed for the sampled rows too -- and thrown away,
    attention reads the given ``k, v [1,T,Hk,D]`` -- so that the timed work is exactly
    ``R/T`` of the full layer's.  Used only as the timed CPU baseline."""
    T, H = x.shape[1], x.shape[2]
    Hq, Hk, D = num_q_heads, num_kv_heads, head_dim
    rows = rows.to(torch.int64)
    R = rows.numel()
    xr = x[0, rows].to(torch.float32)
    am = as_group_mask(attn_mask_rows, 1, R)[0]
    NGa = am.shape[-1]
    q = (xr @ w["wq"].T).view(R, NGa, -1).masked_fill(~am[..., None], 0).view(1, R, Hq, D)
    _ = xr @ w["wk"].T, xr @ w["wv"].T
    # dense attention over all heads in chunks of rows (bounds the score matrix); a chunk
    # reads the keys up to its last row, as a causal kernel over the full sequence would
    a = torch.empty(R, Hq, D)
    order = torch.argsort(rows)
    for c0 in range(0, R, 256):
        sel = order[c0:c0 + 256]
        kmax = int(rows[sel].max()) + 1
        allow = torch.arange(kmax)[None, :] <= rows[sel][:, None]
        a[sel] = torch.nn.functional.scaled_dot_product_attention(
            q[:, sel].transpose(1, 2), k[:, :kmax].transpose(1, 2), v[:, :kmax].transpose(1, 2),
            attn_mask=allow[None, None], enable_gqa=Hq != Hk).transpose(1, 2)[0]
    a = a.reshape(R, NGa, -1).masked_fill(~am[..., None], 0).reshape(R, Hq * D)
    x1 = xr + a @ w["wo"].T
    return x1[None] + dense_then_mask_ffn(x1[None], w["wg"], w["wu"], w["wd"], ffn_mask_rows)


# ----------------------------------------------------------------------------
# error metric
# ----------------------------------------------------------------------------

def rel_err(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """max|actual-expected| / rms(expected): the tolerance is stated on this."""
    e = expected.to(torch.float32)
    a = actual.to(torch.float32).reshape(e.shape)
    rms = float(torch.sqrt(torch.mean(e * e)))
    if rms == 0.0:
        return float((a - e).abs().max())
    return float((a - e).abs().max()) / rms


def rel_err_active(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """max|err| / rms over the entries the routing left non-zero.

    Routed-out blocks are exact zeros on both sides; counting them in the RMS would
    only shrink the denominator by the keep ratio and turn the half-ulp of a bf16
    output (2^-8 relative) into an apparent error above the tolerance.
    """
    e = expected.to(torch.float32)
    a = actual.to(torch.float32).reshape(e.shape)
    nz = e != 0
    if not bool(nz.any()):
        return float((a - e).abs().max()) if e.numel() else 0.0
    rms = float(torch.sqrt(torch.mean(e[nz] * e[nz])))
    return float((a - e).abs().max()) / rms


def rel_err_rows(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """max over rows (last dimension) of max|err| / rms(row), ignoring all-zero rows.

    Attention rows live on very different scales (a causal row that sees one key is
    a copy of a V row, a row that sees thousands is an average close to zero), so a
    single global RMS would charge the output rounding of the large rows against
    the scale of the small ones.
    """
    e = expected.to(torch.float32)
    a = actual.to(torch.float32).reshape(e.shape)
    e2 = e.reshape(-1, e.shape[-1])
    a2 = a.reshape(-1, e.shape[-1])
    rms = torch.sqrt(torch.mean(e2 * e2, dim=-1))
    err = (a2 - e2).abs().max(dim=-1).values
    live = rms > 0
    worst_dead = float(err[~live].max()) if bool((~live).any()) else 0.0
    if worst_dead > 0:
        return float("inf")
    return float((err[live] / rms[live]).max()) if bool(live.any()) else 0.0
