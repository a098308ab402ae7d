"""Dynamic-width SwiGLU FFN with a pre-allocated workspace.

``RoutedFFN`` is the allocation-free form of :func:`dpk_b200.ops.ffn_swiglu`: the
routing layout, packed routing bits and the intermediate activation live in buffers
created once, so a forward call only enqueues kernels (route compaction, bit
packing, fused gate/up projection, down projection) on the current stream.  It is
what a model wrapper keeps per layer, and what the benchmark times.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch

from . import _native as N
from .ops import _dtype_code, _mask_bytes, _need_cuda, _stream


class RoutedFFN:
    """``y = down( mask * silu(gate(x)) * up(x) )`` for ``[M,H]`` tokens.

    Weights: ``gate_weight, up_weight [I,H]``, ``down_weight [H,I]`` (a slice of the
    full matrices under tensor parallelism), ``num_groups`` routed groups of
    ``I/num_groups`` channels.  Same mathematics as the reference callers'
    ``gemm_mn(silu) * gemm_mn -> gemm_k`` (``PruningInferSim/ops/mlp/m_pruning.py:
    76-105``; ``WIDE/wrapper/attn_group_ffn_block.py:33-38``).
    """

    def __init__(self, gate_weight: torch.Tensor, up_weight: torch.Tensor,
                 down_weight: torch.Tensor, num_groups: int, max_tokens: int):
        dev = _need_cuda(gate_weight, up_weight, down_weight)
        self.code = _dtype_code(gate_weight)
        I, H = gate_weight.shape
        if up_weight.shape != (I, H) or down_weight.shape != (H, I):
            raise ValueError("weight shapes must be [I,H], [I,H], [H,I]")
        if I % num_groups:
            raise ValueError(f"I={I} is not divisible by num_groups={num_groups}")
        self.H, self.I, self.NG, self.max_tokens = H, I, num_groups, max_tokens
        self.wg, self.wu, self.wd = (w.contiguous() for w in (gate_weight, up_weight, down_weight))
        self.device = dev
        self.lib = N.load()
        M, NG = max_tokens, num_groups
        words = (NG + 31) // 32
        u8, i32, i64 = torch.uint8, torch.int32, torch.int64
        self.sorted_mask = torch.empty((M, NG), dtype=u8, device=dev)
        self.sorted_indices = torch.empty((M, NG), dtype=i64, device=dev)
        self.counts = torch.empty((NG,), dtype=i32, device=dev)
        self.route_ws_bytes = self.lib.dpk_route_workspace_bytes(1, M, NG)
        self.route_ws = torch.empty(max(self.route_ws_bytes, 16), dtype=u8, device=dev)
        self.row_bits = torch.empty((M, words), dtype=i32, device=dev)
        self.win_bits = torch.empty(((M + 127) // 128, words), dtype=i32, device=dev)
        self.h = torch.empty((M, I), dtype=gate_weight.dtype, device=dev)
        self.acc_bytes = self.lib.dpk_gemm_k_workspace_bytes(M, H)
        self.acc = torch.empty(max(self.acc_bytes, 16), dtype=u8, device=dev)
        self.launches_per_call = 3 + 1 + 1       # routing plan (3 kernels), gate/up, down
        # decode-sized calls (at most 128 tokens): two launches, no routing layout; the workspace
        # is zero-filled here once and left zero by every call
        self.small_tokens = 128 if (H % 128 == 0 and I % 128 == 0) else 0
        self.small_ws = None
        if self.small_tokens:
            n = self.lib.dpk_ffn_small_workspace_bytes(min(max_tokens, 128), H, I)
            self.small_ws = torch.zeros(n, dtype=u8, device=dev)
        # tensor-parallel ranks: a dpk_b200.peer.RowParallelSum of width H makes the down
        # projection store its partial sums into the owners' memory and return the summed y
        self.row_parallel = None

    def __call__(self, x: torch.Tensor, mask: torch.Tensor, out: Optional[torch.Tensor] = None,
                 events: Optional[Dict[str, List[Tuple[torch.cuda.Event, torch.cuda.Event]]]] = None,
                 row_chunks: int = 1,
                 chunk_done: Optional[Callable[[torch.Tensor], None]] = None,
                 residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x``: ``[..., H]``; ``mask``: ``[..., NG]`` (bool / 0-1).  When ``events``
        is a dict, CUDA event pairs bracketing the two GEMM kernels are appended to
        ``events["gemm_mn"]`` and ``events["gemm_k"]``.

        ``row_chunks > 1`` runs the down projection in that many token chunks (multiples
        of 128 rows) and calls ``chunk_done(y_rows)`` after each launch -- the hook a
        tensor-parallel caller uses to start the all-reduce of a finished chunk while the
        next one is being computed.

        ``residual [..., H]``: added to the result in the down projection's epilogue (fp32, one
        rounding): the skip connection of the sub-block without a pass of its own.

        With ``self.row_parallel`` set the down projection is the fused row-parallel sum
        instead: the result (plus ``residual`` when given) is the sum over the
        ranks, returned as a view of the shared output buffer."""
        lead = x.shape[:-1]
        xf = x.reshape(-1, self.H)
        if not xf.is_contiguous():
            xf = xf.contiguous()
        M = xf.shape[0]
        if M > self.max_tokens:
            raise ValueError(f"{M} tokens exceed the planned maximum {self.max_tokens}")
        if out is not None and self.row_parallel is not None:
            raise ValueError("out= cannot be given with a row-parallel sum: the summed result lives "
                             "in the buffer the ranks share and is returned as a view of it")
        m8 = _mask_bytes(mask.reshape(M, self.NG))
        y = out.view(M, self.H) if out is not None else torch.empty(
            (M, self.H), dtype=xf.dtype, device=self.device)
        lib, st, ck = self.lib, _stream(), N.check
        H, I, NG = self.H, self.I, self.NG
        if 0 < M <= self.small_tokens and self.row_parallel is None and residual is None:    # decode-sized
            ev = None
            if events is not None:
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                ev[0].record()
            ck(lib.dpk_ffn_swiglu_small(xf.data_ptr(), self.wg.data_ptr(), self.wu.data_ptr(),
                                        self.wd.data_ptr(), m8.data_ptr(), y.data_ptr(), M, H, I, NG,
                                        self.code, self.small_ws.data_ptr(), self.small_ws.numel(), st))
            if ev is not None:
                ev[1].record()
                events.setdefault("gemm_mn", []).append((ev[0], ev[1]))     # both launches
                events.setdefault("gemm_k", []).append((ev[1], ev[1]))
            if chunk_done is not None:
                chunk_done(y)
            return y.reshape(*lead, self.H)
        ck(lib.dpk_route_plan(m8.data_ptr(), M, NG, self.sorted_mask.data_ptr(),
                              self.sorted_indices.data_ptr(), self.counts.data_ptr(),
                              self.row_bits.data_ptr(), self.win_bits.data_ptr(),
                              self.route_ws.data_ptr(), self.route_ws_bytes, st))
        ev = None
        if events is not None:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record()
        ck(lib.dpk_gemm_mn(xf.data_ptr(), H, self.wg.data_ptr(), self.wu.data_ptr(), H,
                           self.sorted_indices.data_ptr(), self.counts.data_ptr(), self.h.data_ptr(),
                           I, M, I, H, NG, self.code, 0, st))
        if ev is not None:
            ev[1].record()
            ev[2].record()
        if self.row_parallel is not None:
            res2 = residual.reshape(M, H) if residual is not None else None
            ysum = self.row_parallel.gemm_k(self.h[:M], self.wd, self.row_bits, self.win_bits, NG,
                                            residual=res2)
            if ev is not None:
                ev[3].record()
                events.setdefault("gemm_mn", []).append((ev[0], ev[1]))
                events.setdefault("gemm_k", []).append((ev[2], ev[3]))
            return ysum.view(*lead, H)
        res2 = None
        if residual is not None:
            res2 = residual.reshape(M, H)
            if res2.stride(-1) != 1 or res2.stride(0) % 8 or res2.dtype != y.dtype:
                raise ValueError("residual must be a [.., H] tensor of the output's dtype with 16-byte aligned rows")
        words = self.row_bits.shape[1]
        step = M if row_chunks <= 1 else max(128, ((M + row_chunks - 1) // row_chunks + 127) // 128 * 128)
        esz = y.element_size()
        for r0 in range(0, M, step):
            rows = min(step, M - r0)
            ck(lib.dpk_gemm_k(self.h.data_ptr() + r0 * I * esz, I, self.wd.data_ptr(), I,
                              self.row_bits.data_ptr() + r0 * words * 4,
                              self.win_bits.data_ptr() + (r0 // 128) * words * 4,
                              y.data_ptr() + r0 * H * esz, H, rows, H, I, NG, self.code,
                              res2.data_ptr() + r0 * res2.stride(0) * esz if res2 is not None else None,
                              res2.stride(0) if res2 is not None else 0,
                              self.acc.data_ptr() if self.acc_bytes else None, self.acc_bytes, st))
            if chunk_done is not None:
                chunk_done(y[r0:r0 + rows])
        if ev is not None:
            ev[3].record()
            events.setdefault("gemm_mn", []).append((ev[0], ev[1]))
            events.setdefault("gemm_k", []).append((ev[2], ev[3]))
        return y.reshape(*lead, self.H)
