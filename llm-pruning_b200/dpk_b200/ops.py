"""Host-side operators with the reference's call signatures, backed by the C ABI.

Each function mirrors the host wrapper of one reference family (same argument
names, meaning, asserts and return values) and forwards raw pointers to
``libdpk_b200.so``.  Tuning keywords of the reference's JIT path (``autotune``,
``cudagraph``, ``estimate_sparsity``, ``kernel_version``, ``arch``) are accepted
and ignored: the kernels are compiled ahead of time.  CPU tensors are rejected;
there is no fallback path.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _native as N

_GEMV_MN_MAX_M = 4   # reference: python/gemm_mn/jit.py:41


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return N.BF16
    if t.dtype == torch.float16:
        return N.F16
    raise ValueError(f"dpk_b200 kernels take float16 or bfloat16 tensors, got {t.dtype}")


def _need_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("dpk_b200 operators run on CUDA tensors only (no CPU fallback)")
        if t.device != dev:
            raise ValueError("all tensors must be on the same device")
    return dev


def _mask_bytes(mask: torch.Tensor) -> torch.Tensor:
    """Any-dtype 0/1 mask -> contiguous uint8 view/copy (non-zero = active)."""
    if mask.dtype == torch.bool:
        m = mask.contiguous().view(torch.uint8)
    elif mask.dtype == torch.uint8:
        m = mask.contiguous()
    else:
        m = (mask != 0).contiguous().view(torch.uint8)
    return m


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _heads_view(t: torch.Tensor) -> Tuple[torch.Tensor, int, int]:
    """``t [B,T,heads,D]`` as the kernels address it: the heads of a token back to back, token
    and batch strides free (multiples of 8 elements, 16-byte aligned base).  Returns
    ``(tensor, token_stride, batch_stride)`` in elements, copying only a tensor that does not
    fit -- a slice of a fused projection's output or the first rows of a KV cache with spare
    capacity is read in place."""
    B, T, Hh, D = t.shape
    heads_packed = t.stride(3) == 1 and (Hh == 1 or t.stride(2) == D)
    ts = t.stride(1) if T > 1 else Hh * D          # a stride over a dimension of one is never used
    bs = t.stride(0) if B > 1 else T * ts
    if not (heads_packed and ts >= Hh * D and ts % 8 == 0 and bs % 8 == 0 and t.data_ptr() % 16 == 0):
        t = t.contiguous()
        ts, bs = Hh * D, T * Hh * D
    return t, ts, bs


# --------------------------------------------------------------------------- routing

def topk_route_mask(logits: torch.Tensor, keep: int) -> torch.Tensor:
    """Bool mask keeping each token's ``keep`` largest router logits (ties to the
    lower group index).  ``logits``: ``[..., NG]`` float32 on CUDA."""
    _need_cuda(logits)
    l32 = logits.to(torch.float32).contiguous()
    NG = l32.shape[-1]
    M = l32.numel() // NG
    mask = torch.empty(l32.shape, dtype=torch.uint8, device=l32.device)
    with torch.cuda.device(l32.device):
        N.check(N.load().dpk_topk_mask(l32.data_ptr(), M, NG, int(keep), mask.data_ptr(), _stream()))
    return mask.view(torch.bool)


def router_norm(x: torch.Tensor, w_down: torch.Tensor, b_down: Optional[torch.Tensor],
                w_route: torch.Tensor, b_route: Optional[torch.Tensor],
                norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                return_logits: bool = False, round_like_module: bool = True):
    """Two-stage token router, its evaluation-time decision and (optionally) the RMSNorm of
    the same hidden state, in one pass over ``x [..., H]``.

    Mirrors ``TokenRouter.forward`` followed by the eval branch of ``_gumbel_softmax``
    (``WIDE/wrapper/base_layer.py:89-114, 204-207``) and the layer norm called next to it
    (``WIDE/wrapper/attn_group_ffn_block.py:170-176``).  Returns ``(execute bool [..., NG],
    xn [..., H] or None, logits float32 [..., NG, 2] or None)``."""
    dev = _need_cuda(x, w_down, w_route, b_down, b_route, norm_weight)
    code = _dtype_code(x)
    lead, H = x.shape[:-1], x.shape[-1]
    x2 = x.reshape(-1, H)
    if x2.stride(-1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    M = x2.shape[0]
    R = w_down.shape[0]
    if w_down.shape != (R, H) or w_route.shape[1] != R or w_route.shape[0] % 2:
        raise ValueError("w_down must be [R,H] and w_route [2*NG,R]")
    NG = w_route.shape[0] // 2
    for t in (w_down, w_route, b_down, b_route, norm_weight):
        if t is not None and t.dtype != x.dtype:
            raise ValueError("router and norm parameters must have the dtype of x")
    wd, wr = w_down.contiguous(), w_route.contiguous()
    execute = torch.empty((M, NG), dtype=torch.uint8, device=dev)
    xn = torch.empty((M, H), dtype=x.dtype, device=dev) if norm_weight is not None else None
    logits = torch.empty((M, NG, 2), dtype=torch.float32, device=dev) if return_logits else None
    with torch.cuda.device(dev):
        N.check(N.load().dpk_router_norm(
            x2.data_ptr(), x2.stride(0), _ptr(norm_weight.contiguous() if norm_weight is not None else None),
            float(eps), wd.data_ptr(), _ptr(b_down.contiguous() if b_down is not None else None),
            wr.data_ptr(), _ptr(b_route.contiguous() if b_route is not None else None), _ptr(xn), H,
            execute.data_ptr(), _ptr(logits), M, H, R, NG, code, 1 if round_like_module else 0,
            _stream()))
    return (execute.view(*lead, NG).bool(), xn.view(*lead, H) if xn is not None else None,
            logits.view(*lead, NG, 2) if logits is not None else None)


def rope_append(q: torch.Tensor, k: torch.Tensor, v: Optional[torch.Tensor], cos: torch.Tensor,
                sin: torch.Tensor, k_cache: Optional[torch.Tensor] = None,
                v_cache: Optional[torch.Tensor] = None, past_len: int = 0):
    """Rotary embedding of ``q [B,T,Hq,D]`` and ``k [B,T,Hk,D]`` (in place) and, when the
    caches ``[B,capacity,Hk,D]`` are given, the append of the rotated ``k`` and of ``v`` at
    ``past_len``.  ``cos, sin``: ``[T,D]``, ``[1,T,D]`` or ``[B,T,D]``.  Mirrors
    ``apply_rotary_pos_emb`` + ``past_key_values.update`` of the reference's attention wrapper
    (``WIDE/wrapper/attn_group_ffn_block.py:60-67``).  Returns ``(q, keys, values)`` where
    ``keys, values`` are the first ``past_len+T`` cache rows (or ``k, v`` without a cache)."""
    dev = _need_cuda(q, k, v, cos, sin, k_cache, v_cache)
    code = _dtype_code(q)
    B, T, Hq, D = q.shape
    Hk = k.shape[2]
    if k.shape != (B, T, Hk, D) or (v is not None and v.shape != k.shape):
        raise ValueError("q, k, v must be [B,T,heads,D] with equal B, T, D")
    def flat_stride(t, heads):
        # tokens of all batch entries one stride apart: [B*T, width] rows with the heads packed
        ok = (t.stride(3) == 1 and (heads == 1 or t.stride(2) == D) and t.stride(1) % 8 == 0
              and t.stride(1) >= heads * D and (B == 1 or t.stride(0) == T * t.stride(1)))
        if not ok:
            raise ValueError("q, k, v must keep a token's heads back to back and all tokens one stride "
                             "apart (q and k are rotated in place, so no copy is made)")
        return t.stride(1)
    q_ts, kv_ts = flat_stride(q, Hq), flat_stride(k, Hk)
    if v is not None and flat_stride(v, Hk) != kv_ts:
        raise ValueError("k and v must share one token stride")
    if cos.dim() == 2:
        cos, sin = cos[None], sin[None]
    if cos.shape[-2:] != (T, D) or sin.shape != cos.shape or cos.shape[0] not in (1, B):
        raise ValueError("cos and sin must be [T,D], [1,T,D] or [B,T,D]")
    cos, sin = cos.contiguous(), sin.contiguous()
    if cos.dtype != q.dtype or sin.dtype != q.dtype or k.dtype != q.dtype:
        raise ValueError("q, k, cos and sin must share one dtype")
    stride = 0 if cos.shape[0] == 1 else T * D
    capacity = 0
    if k_cache is not None:
        if v_cache is None or v is None:
            raise ValueError("k_cache needs v_cache and v")
        capacity = k_cache.shape[1]
        want = (B, capacity, Hk, D)
        if k_cache.shape != want or v_cache.shape != want or not (
                k_cache.is_contiguous() and v_cache.is_contiguous()):
            raise ValueError("caches must be contiguous [B,capacity,Hk,D]")
    with torch.cuda.device(dev):
        N.check(N.load().dpk_rope_append(q.data_ptr(), k.data_ptr(), _ptr(v), cos.data_ptr(),
                                         sin.data_ptr(), stride, _ptr(k_cache), _ptr(v_cache), B, T,
                                         Hq, Hk, D, capacity, past_len, code, q_ts, kv_ts, _stream()))
    if k_cache is None:
        return q, k, v
    return q, k_cache[:, :past_len + T], v_cache[:, :past_len + T]


def route_compact(mask: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Routing layout of a ``[M,NG]`` or ``[B,M,NG]`` mask (sorted per batch).

    Returns ``(sorted_mask bool, sorted_indices int64, counts int32[(B,)NG])`` with
    the active rows of every group column first, in ascending order -- what the
    reference builds with ``torch.sort(mask, descending=True)``
    (``python/gemm_mn/jit.py:410-415``, ``python/attention_prefill/jit.py:259-263``).
    """
    _need_cuda(mask)
    m8 = _mask_bytes(mask)
    if m8.dim() == 2:
        batches, (M, NG) = 1, m8.shape
    elif m8.dim() == 3:
        batches, M, NG = m8.shape
    else:
        raise ValueError("mask must be [M,NG] or [B,M,NG]")
    dev = m8.device
    smask = torch.empty(m8.shape, dtype=torch.uint8, device=dev)
    sidx = torch.empty(m8.shape, dtype=torch.int64, device=dev)
    counts = torch.empty(m8.shape[:-2] + (NG,), dtype=torch.int32, device=dev)
    lib = N.load()
    nbytes = lib.dpk_route_workspace_bytes(batches, M, NG)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        N.check(lib.dpk_route_compact(m8.data_ptr(), batches, M, NG, smask.data_ptr(),
                                      sidx.data_ptr(), counts.data_ptr(), ws.data_ptr(), nbytes,
                                      _stream()))
    return smask.view(torch.bool), sidx, counts


def _counts_of(sorted_mask: torch.Tensor) -> torch.Tensor:
    sm8 = _mask_bytes(sorted_mask)
    if sm8.dim() == 2:
        batches, (M, NG) = 1, sm8.shape
    else:
        batches, M, NG = sm8.shape
    counts = torch.empty(sm8.shape[:-2] + (NG,), dtype=torch.int32, device=sm8.device)
    with torch.cuda.device(sm8.device):
        N.check(N.load().dpk_route_counts(sm8.data_ptr(), batches, M, NG, counts.data_ptr(),
                                          _stream()))
    return counts


def _layout_for(mask3: torch.Tensor, sorted_mask, sorted_indices, shape):
    """Return (sorted_mask, sorted_indices, counts) viewed as ``shape``, computing the
    layout when the caller did not pass one."""
    if sorted_indices is None:
        return route_compact(mask3.reshape(shape))
    if sorted_mask is None:
        raise ValueError("sorted_mask must accompany sorted_indices")
    smask = sorted_mask.reshape(shape)
    sidx = sorted_indices.reshape(shape)
    if sidx.dtype != torch.int64:
        raise ValueError("sorted_indices must be int64")
    sidx = sidx.contiguous()
    return smask, sidx, _counts_of(smask)


# --------------------------------------------------------------------- routed GEMMs

def gemm_mn(A: torch.Tensor, B: torch.Tensor, Mask: torch.Tensor, D: Optional[torch.Tensor] = None,
            sorted_mask: Optional[torch.Tensor] = None,
            sorted_indices: Optional[torch.Tensor] = None, activation: Optional[str] = "identity",
            estimate_sparsity: Optional[float] = 0.5, kernel_version: Optional[int] = 0,
            arch: Optional[str] = "sm100", autotune: Optional[bool] = True, cudagraph: bool = False,
            up_weight: Optional[torch.Tensor] = None):
    """Output-width routed projection; signature of the reference's ``gemm_mn``
    (``python/gemm_mn/jit.py:357-440``).  Returns ``(D[B,T,N], metadata)``.

    ``up_weight`` (extension): a second ``[N,K]`` weight; the result is then
    ``silu(A B^T) * (A up_weight^T)`` computed in one pass.
    """
    assert A.dim() == 3 and B.dim() == 2
    assert Mask.dim() in (2, 3)
    assert estimate_sparsity <= 1
    dev = _need_cuda(A, B, Mask, D, up_weight)
    code = _dtype_code(A)
    if B.dtype != A.dtype or (up_weight is not None and up_weight.dtype != A.dtype):
        raise ValueError("A and the weights must share one dtype")
    if activation not in N.ACT:
        raise ValueError(f"Unsupported activation: {activation}")
    Bsz, T, K = A.shape
    A_f = A.flatten(0, 1)
    if A_f.stride(-1) != 1 or A_f.stride(0) % 8:
        A_f = A_f.contiguous()
    M = A_f.shape[0]
    Nw = B.shape[0]
    if B.shape[1] != K:
        raise ValueError("A and B disagree on K")
    Bc = B if B.stride(-1) == 1 and B.stride(0) % 8 == 0 else B.contiguous()
    Uc = None
    if up_weight is not None:
        if up_weight.shape != B.shape:
            raise ValueError("up_weight must have the shape of B")
        Uc = up_weight.contiguous()
        Bc = Bc.contiguous()
    if D is None:
        D = torch.zeros((M, Nw), dtype=A.dtype, device=dev)
    D2 = D.view(M, Nw)
    if Mask.dim() == 2:
        Mask = Mask.unsqueeze(-1)
    NG = Mask.shape[-1]
    if Nw % NG:
        raise ValueError(f"Output width {Nw} must be divisible by groups {NG}")
    G = Nw // NG
    lib = N.load()
    metadata: Dict[str, torch.Tensor] = {}
    with torch.cuda.device(dev):
        use_gemv = M <= _GEMV_MN_MAX_M and up_weight is None
        tensor_core_ok = G % 16 == 0 and K % 8 == 0
        if use_gemv or not tensor_core_ok:
            if up_weight is not None:
                raise ValueError("the fused SwiGLU path needs G % 16 == 0 and K % 8 == 0")
            m8 = _mask_bytes(Mask.flatten(0, 1))
            N.check(lib.dpk_gemv_routed(A_f.data_ptr(), A_f.stride(0), Bc.data_ptr(), Bc.stride(0),
                                        m8.data_ptr(), D2.data_ptr(), D2.stride(0), M, Nw, K, NG,
                                        code, N.ACT[activation], 0, _stream()))
            if not use_gemv:
                smask, sidx, _ = _layout_for(Mask, sorted_mask, sorted_indices, (M, NG))
                metadata = dict(sorted_mask=smask, sorted_indices=sidx)
        else:
            smask, sidx, counts = _layout_for(Mask, sorted_mask, sorted_indices, (M, NG))
            metadata = dict(sorted_mask=smask, sorted_indices=sidx)
            N.check(lib.dpk_gemm_mn(A_f.data_ptr(), A_f.stride(0), Bc.data_ptr(), _ptr(Uc),
                                    Bc.stride(0), sidx.data_ptr(), counts.data_ptr(), D2.data_ptr(),
                                    D2.stride(0), M, Nw, K, NG, code, N.ACT[activation], _stream()))
    return D2.reshape(Bsz, T, Nw), metadata


def _use_gemv_k_dispatch(M: int, G: int) -> bool:
    """Reference rule, ``python/gemm_k/jit.py:337-342``."""
    if M == 1:
        return G >= 256
    if M == 2:
        return G >= 128
    return M == 4 and G >= 64


def gemm_k(A: torch.Tensor, B: torch.Tensor, Mask: torch.Tensor, D: Optional[torch.Tensor] = None,
           sorted_mask: Optional[torch.Tensor] = None, sorted_indices: Optional[torch.Tensor] = None,
           estimate_sparsity: Optional[float] = 0.5, kernel_version: Optional[int] = 0,
           arch: Optional[str] = "sm100", autotune: Optional[bool] = True, cudagraph: bool = False,
           residual: Optional[torch.Tensor] = None):
    """Reduction-width routed projection; signature of the reference's ``gemm_k``
    (``python/gemm_k/jit.py:345-425``).  Returns ``(D[B,T,N], metadata)``; ``D`` is
    overwritten.

    ``residual`` (extension): a ``[B,T,N]`` tensor added to the projection in fp32 before the
    single rounding -- the skip connection of the sub-block in the same pass.  Passing ``D``
    itself gives the accumulate-onto-``D`` behaviour of the reference's CuTe path
    (``python/gemm_k/jit.py:368``)."""
    assert A.dim() == 3 and B.dim() == 2
    assert Mask.dim() in (2, 3)
    assert estimate_sparsity <= 1
    dev = _need_cuda(A, B, Mask, D)
    code = _dtype_code(A)
    if B.dtype != A.dtype:
        raise ValueError("A and B must share one dtype")
    Bsz, T, K = A.shape
    A_f = A.flatten(0, 1)
    if A_f.stride(-1) != 1 or A_f.stride(0) % 8:
        A_f = A_f.contiguous()
    M = A_f.shape[0]
    Nw = B.shape[0]
    if B.shape[1] != K:
        raise ValueError("A and B disagree on K")
    Bc = B if B.stride(-1) == 1 and B.stride(0) % 8 == 0 else B.contiguous()
    if D is None:
        # every path below writes every element of D (rows without an active group come out
        # as zeros, or as the residual), so a fresh output needs no zero-fill
        D = torch.empty((M, Nw), dtype=A.dtype, device=dev)
    D2 = D.view(M, Nw)
    if Mask.dim() == 2:
        Mask = Mask.unsqueeze(-1)
    NG = Mask.shape[-1]
    if K % NG:
        raise ValueError(f"Input width {K} must be divisible by groups {NG}")
    G = K // NG
    lib = N.load()
    m8 = _mask_bytes(Mask.flatten(0, 1))
    metadata: Dict[str, torch.Tensor] = {}
    R2 = None
    if residual is not None:
        if residual.shape[-1] != Nw or residual.numel() != M * Nw or residual.dtype != A.dtype:
            raise ValueError("residual must have the shape and dtype of the output")
        R2 = residual.reshape(M, Nw)
        if R2.stride(-1) != 1 or R2.stride(0) % 8 or R2.data_ptr() % 16:
            R2 = R2.contiguous()
    with torch.cuda.device(dev):
        use_gemv = _use_gemv_k_dispatch(M, G)
        tensor_core_ok = G % 64 == 0 and Nw % 8 == 0
        if (NG == 1 and R2 is None and not use_gemv and M >= 256 and Nw % 16 == 0 and K % 8 == 0
                and D2.is_contiguous()):
            # A whole-token mask (one group spanning all of K; LFF's token gate) is the same
            # product as an output-width routed projection with one group spanning all of N: the
            # active rows are compacted, so no MMA row is spent on a skipped token (the masked
            # kernel below only skips whole 128-token windows).  Skipped rows are zero.
            smask, sidx, counts = _layout_for(Mask, sorted_mask, sorted_indices, (M, NG))
            D2.zero_()
            N.check(lib.dpk_gemm_mn(A_f.data_ptr(), A_f.stride(0), Bc.data_ptr(), None, Bc.stride(0),
                                    sidx.data_ptr(), counts.data_ptr(), D2.data_ptr(), D2.stride(0),
                                    M, Nw, K, 1, code, N.ACT["identity"], _stream()))
            return D2.reshape(Bsz, T, Nw), dict(sorted_mask=smask, sorted_indices=sidx)
        if use_gemv or not tensor_core_ok:
            N.check(lib.dpk_gemv_routed(A_f.data_ptr(), A_f.stride(0), Bc.data_ptr(), Bc.stride(0),
                                        m8.data_ptr(), D2.data_ptr(), D2.stride(0), M, Nw, K, NG,
                                        code, 0, 1, _stream()))
            if R2 is not None:
                D2.add_(R2)                  # the few-row GEMV path has no fused residual
        else:
            words = (NG + 31) // 32
            row_bits = torch.empty((M, words), dtype=torch.int32, device=dev)
            win_bits = torch.empty(((M + 127) // 128, words), dtype=torch.int32, device=dev)
            N.check(lib.dpk_mask_pack(m8.data_ptr(), M, NG, row_bits.data_ptr(),
                                      win_bits.data_ptr(), _stream()))
            nbytes = lib.dpk_gemm_k_workspace_bytes(M, Nw)
            ws = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
            N.check(lib.dpk_gemm_k(A_f.data_ptr(), A_f.stride(0), Bc.data_ptr(), Bc.stride(0),
                                   row_bits.data_ptr(), win_bits.data_ptr(), D2.data_ptr(),
                                   D2.stride(0), M, Nw, K, NG, code, _ptr(R2),
                                   R2.stride(0) if R2 is not None else 0, _ptr(ws), nbytes, _stream()))
        if not use_gemv:
            smask, sidx, _ = _layout_for(Mask, sorted_mask, sorted_indices, (M, NG))
            metadata = dict(sorted_mask=smask, sorted_indices=sidx)
    return D2.reshape(Bsz, T, Nw), metadata


def ffn_swiglu(x: torch.Tensor, gate_weight: torch.Tensor, up_weight: torch.Tensor,
               down_weight: torch.Tensor, Mask: torch.Tensor,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dynamic-width SwiGLU FFN ``down(mask * silu(gate(x)) * up(x))`` in one native
    call.  ``x``: ``[B,T,H]``; weights ``[I,H]``, ``[I,H]``, ``[H,I]``; ``Mask``:
    ``[B,T,NG]`` (or ``[B,T]``).  Equivalent to the reference callers' composition
    of ``gemm_mn`` (silu), ``gemm_mn``, multiply and ``gemm_k``
    (``PruningInferSim/ops/mlp/m_pruning.py:76-105``)."""
    assert x.dim() == 3 and Mask.dim() in (2, 3)
    dev = _need_cuda(x, gate_weight, up_weight, down_weight, Mask, out)
    code = _dtype_code(x)
    Bsz, T, H = x.shape
    I = gate_weight.shape[0]
    if gate_weight.shape != (I, H) or up_weight.shape != (I, H) or down_weight.shape != (H, I):
        raise ValueError("weight shapes must be [I,H], [I,H], [H,I]")
    if Mask.dim() == 2:
        Mask = Mask.unsqueeze(-1)
    NG = Mask.shape[-1]
    M = Bsz * T
    xf = x.reshape(M, H).contiguous()
    wg, wu, wd = gate_weight.contiguous(), up_weight.contiguous(), down_weight.contiguous()
    m8 = _mask_bytes(Mask.flatten(0, 1))
    y = out.view(M, H) if out is not None else torch.empty((M, H), dtype=x.dtype, device=dev)
    lib = N.load()
    if 0 < M <= 128 and H % 128 == 0 and I % 128 == 0 and I % NG == 0:
        # decode-sized call: two launches, no routing layout; the workspace has to start zero
        nbytes = lib.dpk_ffn_small_workspace_bytes(M, H, I)
        with torch.cuda.device(dev):
            ws = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
            N.check(lib.dpk_ffn_swiglu_small(xf.data_ptr(), wg.data_ptr(), wu.data_ptr(),
                                             wd.data_ptr(), m8.data_ptr(), y.data_ptr(), M, H, I, NG,
                                             code, ws.data_ptr(), nbytes, _stream()))
        return y.reshape(Bsz, T, H)
    nbytes = lib.dpk_ffn_workspace_bytes(M, H, I, NG)
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        N.check(lib.dpk_ffn_swiglu(xf.data_ptr(), wg.data_ptr(), wu.data_ptr(), wd.data_ptr(),
                                   m8.data_ptr(), y.data_ptr(), M, H, I, NG, code, ws.data_ptr(),
                                   nbytes, _stream()))
    return y.reshape(Bsz, T, H)


# ------------------------------------------------------------------ routed attention

def _leftpad_arg(Leftpad: Optional[torch.Tensor], B: int, dev) -> Optional[torch.Tensor]:
    if Leftpad is None:
        return None
    lp = Leftpad.to(device=dev)
    if lp.shape != (B,):
        raise ValueError("Leftpad must have shape [batch]")
    return lp.to(torch.int64).to(torch.int32).contiguous()   # same 32 bits as uint32


def _padded_head_dim(D: int) -> int:
    """The kernels are built for head sizes 64 and 128.  The reference's attention accepts every
    multiple of 32 (``include/attention_prefill/v3/sm12x.cuh:88-99``); 32 and 96 run here with
    zero columns appended to q, k and v (dot products and outputs are unchanged, the softmax
    scale stays that of the original size) at the price of the padded copies."""
    if D in (64, 128):
        return D
    if D % 32 or D <= 0 or D > 128:
        raise ValueError(f"head_dim {D} not supported: multiples of 32 up to 128")
    return 64 if D < 64 else 128


def _pad_heads(t: torch.Tensor, Dp: int) -> torch.Tensor:
    return torch.nn.functional.pad(t, (0, Dp - t.shape[-1]))


def attention_prefill(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, Mask: torch.Tensor,
                      Leftpad: Optional[torch.Tensor] = None, O: Optional[torch.Tensor] = None,
                      sorted_mask: Optional[torch.Tensor] = None,
                      sorted_indices: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                      is_causal: Optional[bool] = True, estimate_sparsity: Optional[float] = 0.5,
                      kernel_version: Optional[int] = 0, arch: Optional[str] = "sm100",
                      autotune: Optional[bool] = True, cudagraph: bool = False):
    """Head-group-routed prefill attention; signature of the reference's
    ``attention_head`` (``python/attention_prefill/jit.py:223-284``).  Returns
    ``(O[B,Tq,Hq,D], {"sorted_mask", "sorted_indices"})``."""
    assert Q.dim() == 4 and K.dim() == 4 and V.dim() == 4
    assert K.shape == V.shape
    assert Mask.dim() == 3
    assert estimate_sparsity <= 1
    dev = _need_cuda(Q, K, V, Mask, O)
    code = _dtype_code(Q)
    if K.dtype != Q.dtype or V.dtype != Q.dtype:
        raise ValueError("Q, K and V must share one dtype")
    B, Tq, Hq, D = Q.shape
    _, Tk, Hk, _ = K.shape
    NG = Mask.shape[-1]
    Dp = _padded_head_dim(D)
    if Dp != D:
        Op, meta = attention_prefill(_pad_heads(Q, Dp), _pad_heads(K, Dp), _pad_heads(V, Dp), Mask, Leftpad,
                                     None, sorted_mask, sorted_indices, D ** -0.5 if scale is None else scale,
                                     is_causal, estimate_sparsity, kernel_version, arch, autotune, cudagraph)
        if O is None:
            return Op[..., :D].contiguous(), meta
        O.copy_(Op[..., :D])
        return O, meta
    Qc, q_ts, q_bs = _heads_view(Q)
    Kc, kv_ts, kv_bs = _heads_view(K)
    Vc, v_ts, v_bs = _heads_view(V)
    if (v_ts, v_bs) != (kv_ts, kv_bs):            # the kernel takes one pair of strides for K and V
        Kc, Vc = K.contiguous(), V.contiguous()
        kv_ts, kv_bs = Hk * D, Tk * Hk * D
    if O is None:
        O = torch.zeros((B, Tq, Hq, D), dtype=Q.dtype, device=dev)
    if not O.is_contiguous():
        raise ValueError("O must be contiguous")
    if scale is None:
        scale = D ** -0.5
    lp = _leftpad_arg(Leftpad, B, dev)
    # the reference's PyTorch path aligns the causal mask bottom-right only when a
    # Leftpad is given (python/references.py:123-139)
    shift = (Tk - Tq) if Leftpad is not None else 0
    with torch.cuda.device(dev):
        smask, sidx, counts = _layout_for(Mask, sorted_mask, sorted_indices, (B, Tq, NG))
        N.check(N.load().dpk_attn_prefill(Qc.data_ptr(), Kc.data_ptr(), Vc.data_ptr(),
                                          sidx.data_ptr(), counts.data_ptr(), _ptr(lp),
                                          O.data_ptr(), B, Tq, Tk, Hq, Hk, D, NG, float(scale),
                                          1 if is_causal else 0, shift, code, q_ts, q_bs, kv_ts, kv_bs,
                                          _stream()))
    return O, dict(sorted_mask=smask, sorted_indices=sidx)


def attention_decode(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, Mask: torch.Tensor,
                     Leftpad: Optional[torch.Tensor] = None, O: Optional[torch.Tensor] = None,
                     sorted_mask: Optional[torch.Tensor] = None,
                     sorted_indices: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                     is_causal: Optional[bool] = True, estimate_sparsity: Optional[float] = 0.5,
                     kernel_version: Optional[int] = 0, arch: Optional[str] = "sm100",
                     autotune: Optional[bool] = True, cudagraph: bool = False):
    """Head-group-routed decode attention; signature of the reference's decode
    ``attention_head`` (``python/attention_decode/jit.py:201-261``).  Returns
    ``(O[B,1,Hq,D], {})``.  One query token attends every cached key, so
    ``is_causal`` has no effect (as in the reference kernel)."""
    assert Q.dim() == 4 and K.dim() == 4 and V.dim() == 4
    assert Q.shape[1] == 1
    assert K.shape == V.shape
    assert Mask.dim() == 3
    assert estimate_sparsity <= 1
    dev = _need_cuda(Q, K, V, Mask, O)
    code = _dtype_code(Q)
    if K.dtype != Q.dtype or V.dtype != Q.dtype:
        raise ValueError("Q, K and V must share one dtype")
    B, _, Hq, D = Q.shape
    _, Tk, Hk, _ = K.shape
    NG = Mask.shape[-1]
    Dp = _padded_head_dim(D)
    if Dp != D:
        Op, meta = attention_decode(_pad_heads(Q, Dp), _pad_heads(K, Dp), _pad_heads(V, Dp), Mask, Leftpad,
                                    None, sorted_mask, sorted_indices, D ** -0.5 if scale is None else scale,
                                    is_causal, estimate_sparsity, kernel_version, arch, autotune, cudagraph)
        if O is None:
            return Op[..., :D].contiguous(), meta
        O.copy_(Op[..., :D])
        return O, meta
    Qc = Q.contiguous()
    Kc, kv_ts, kv_bs = _heads_view(K)
    Vc, v_ts, v_bs = _heads_view(V)
    if (v_ts, v_bs) != (kv_ts, kv_bs):
        Kc, Vc = K.contiguous(), V.contiguous()
        kv_ts, kv_bs = Hk * D, Tk * Hk * D
    if O is None:
        O = torch.empty((B, 1, Hq, D), dtype=Q.dtype, device=dev)
    if not O.is_contiguous():
        raise ValueError("O must be contiguous")
    if scale is None:
        scale = D ** -0.5
    lp = _leftpad_arg(Leftpad, B, dev)
    m8 = _mask_bytes(Mask.reshape(B, NG))
    lib = N.load()
    nbytes = lib.dpk_attn_decode_workspace_bytes(B, Tk, Hq, Hk, D, NG)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        N.check(lib.dpk_attn_decode(Qc.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), m8.data_ptr(),
                                    _ptr(lp), O.data_ptr(), B, Tk, Hq, Hk, D, NG, float(scale), code,
                                    kv_ts, kv_bs, ws.data_ptr(), nbytes, _stream()))
    return O, dict()


def device_status() -> int:
    """Synchronise the current stream and return the kernels' status word."""
    return N.device_status(_stream())
