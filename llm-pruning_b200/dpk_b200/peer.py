"""Row-parallel sum fused into the reduction-width projection (tensor-parallel ranks).

Under the split the reference sketches for its wrappers (down / o projections row
parallel, ``WIDE/transformer_fsdp_hook.py:44-54``) every rank ends a sub-block with a
partial ``[M,N]`` sum that has to be added over the ranks.  Instead of writing the partial
sums to local memory and handing them to an all-reduce, the projection kernel stores each
128-token window straight into the memory of the rank that owns those rows while the other
tiles are still being computed; each owner then adds the slabs it received (fp32, optional
residual) and stores the finished rows into every rank's output.  Between the two kernels,
and after the second, the ranks meet at a barrier (a one-element all-reduce, ordered on
the stream) -- no kernel waits on another GPU.

Buffers come from the C library (``dpk_peer_alloc``) and are mapped into the peers with
CUDA IPC; the 64-byte handles travel through ``torch.distributed``.

:func:`RowParallelSum.emulate` builds the ``world`` ranks inside one process on one GPU
(plain device tensors instead of mapped peer buffers, no barrier needed because one stream
orders everything): the index arithmetic of both kernels is identical, which is what the
single-GPU parity tests exercise.
"""

from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import _native as N
from .ops import _mask_bytes, _stream

MAX_WORLD = 8
WINDOW = 128


def rows_per_owner(M: int, world: int) -> int:
    """Token rows each rank owns: an equal share rounded up to whole 128-token windows."""
    if world < 1 or world > MAX_WORLD:
        raise ValueError(f"world must be 1..{MAX_WORLD}")
    share = (max(M, 1) + world - 1) // world
    return (share + WINDOW - 1) // WINDOW * WINDOW


def owner_of_row(row: int, M: int, world: int) -> int:
    return row // rows_per_owner(M, world)


def slab_offset(row: int, M: int, world: int, source_rank: int, ld: int) -> int:
    """Element offset, inside the owner's staging buffer, of ``row`` as sent by
    ``source_rank`` (layout ``[world, rows_per_owner, ld]``)."""
    R = rows_per_owner(M, world)
    return (source_rank * R + row % R) * ld


class _DeviceBytes:
    """Exposes a raw device allocation to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2, "strides": None}


def _ptr_table(ptrs: Sequence[int]):
    return (C.c_void_p * len(ptrs))(*ptrs)


class RowParallelSum:
    """One fused row-parallel sum of ``[max_rows, width]`` outputs.

    ``gemm_k(...)`` / ``routed_gemm_k(...)`` return this rank's copy of the summed output
    (a view into the peer-visible buffer, valid until the next call).
    """

    def __init__(self, world: int, rank: int, max_rows: int, width: int, dtype: torch.dtype,
                 device: torch.device, stage: torch.Tensor, out: torch.Tensor,
                 stage_ptrs: Sequence[int], out_ptrs: Sequence[int],
                 barrier: Callable[[], None], keep=()):
        self.world, self.rank, self.max_rows, self.width = world, rank, max_rows, width
        self.dtype, self.device = dtype, device
        self.stage, self.out = stage, out
        self._stage_tab, self._out_tab = _ptr_table(stage_ptrs), _ptr_table(out_ptrs)
        self._barrier = barrier
        self._keep = keep
        self.lib = N.load()
        self.code = 1 if dtype == torch.bfloat16 else 0
        self._ws = None
        self.timers = None      # dict -> lists of CUDA events at the five points of a fused sum

    # ---- construction -----------------------------------------------------------------
    @staticmethod
    def _sizes(world: int, max_rows: int, width: int):
        R = rows_per_owner(max_rows, world)
        return R, world * R * width * 2

    @classmethod
    def connect(cls, max_rows: int, width: int, dtype: torch.dtype, device: torch.device,
                group: Optional[dist.ProcessGroup] = None) -> "RowParallelSum":
        """Collective over ``group``: allocate this rank's buffers, exchange the IPC
        handles, map the peers'."""
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        _, nbytes = cls._sizes(world, max_rows, width)
        lib = N.load()
        with torch.cuda.device(device):
            base = C.c_void_p()
            handle = C.create_string_buffer(64)
            N.check(lib.dpk_peer_alloc(2 * nbytes, C.byref(base), handle))
            handles: List[bytes] = [b""] * world
            dist.all_gather_object(handles, handle.raw, group=group)
            bases = []
            for r in range(world):
                if r == rank:
                    bases.append(base.value)
                else:
                    p = C.c_void_p()
                    N.check(lib.dpk_peer_open(handles[r], C.byref(p)))
                    bases.append(p.value)
            raw = torch.as_tensor(_DeviceBytes(base.value, 2 * nbytes), device=device)
        stage = raw[:nbytes].view(dtype)
        out = raw[nbytes:].view(dtype)
        token = torch.zeros(1, device=device)

        def barrier():
            dist.all_reduce(token, group=group)

        return cls(world, rank, max_rows, width, dtype, device, stage, out, bases,
                   [b + nbytes for b in bases], barrier, keep=(raw, token))

    @classmethod
    def emulate(cls, world: int, max_rows: int, width: int, dtype: torch.dtype,
                device: torch.device) -> List["RowParallelSum"]:
        """All ``world`` ranks in this process, on one device."""
        _, nbytes = cls._sizes(world, max_rows, width)
        raws = [torch.empty(2 * nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
        bases = [t.data_ptr() for t in raws]
        return [cls(world, r, max_rows, width, dtype, device, raws[r][:nbytes].view(dtype),
                    raws[r][nbytes:].view(dtype), bases, [b + nbytes for b in bases],
                    lambda: None, keep=tuple(raws)) for r in range(world)]

    # ---- the two halves ---------------------------------------------------------------
    def scatter(self, A2: torch.Tensor, W: torch.Tensor, row_bits: torch.Tensor,
                win_bits: torch.Tensor, NG: int) -> None:
        """First half: this rank's partial sums go to the owners' staging buffers."""
        M, K = A2.shape
        if M > self.max_rows or W.shape != (self.width, K):
            raise ValueError("shape outside what this RowParallelSum was built for")
        R = rows_per_owner(M, self.world)
        need = self.lib.dpk_gemm_k_scatter_workspace_bytes(M, self.width, self.width)
        if need and (self._ws is None or self._ws.numel() < need):
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        N.check(self.lib.dpk_gemm_k_scatter(
            A2.data_ptr(), A2.stride(0), W.data_ptr(), W.stride(0), row_bits.data_ptr(),
            win_bits.data_ptr(), self._stage_tab, self.world, self.rank, R, self.width, M,
            self.width, K, NG, self.code, self._ws.data_ptr() if need else None, need, _stream()))

    def reduce(self, M: int, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Second half: sum the received slabs of the rows this rank owns and store them
        into every rank's output."""
        R = rows_per_owner(M, self.world)
        if residual is not None and (residual.shape != (M, self.width) or not residual.is_contiguous()):
            raise ValueError("residual must be a contiguous [M, width] tensor")
        N.check(self.lib.dpk_reduce_gather(
            self.stage.data_ptr(), self._out_tab, residual.data_ptr() if residual is not None else None,
            self.world, self.rank, R, M, self.width, self.width, self.code, _stream()))
        return self.out[:M * self.width].view(M, self.width)

    def gemm_k(self, A2: torch.Tensor, W: torch.Tensor, row_bits: torch.Tensor,
               win_bits: torch.Tensor, NG: int, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        self._mark("start")
        self.scatter(A2, W, row_bits, win_bits, NG)
        self._mark("scatter")
        self._barrier()          # every rank's partial sums have landed
        self._mark("barrier1")
        y = self.reduce(A2.shape[0], residual)
        self._mark("reduce")
        self._barrier()          # every owner's rows have landed; staging may be reused
        self._mark("barrier2")
        return y

    def _mark(self, name: str) -> None:
        if self.timers is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.timers.setdefault(name, []).append(ev)

    def phase_ms(self) -> dict:
        """Mean milliseconds of the four phases since ``timers`` was set to a dict."""
        names = ["start", "scatter", "barrier1", "reduce", "barrier2"]
        tm = self.timers or {}
        if not tm.get("start"):
            return {}
        return {b + "_ms": sum(e0.elapsed_time(e1) for e0, e1 in zip(tm[a], tm[b])) / len(tm[a])
                for a, b in zip(names[:-1], names[1:])}

    def routed_gemm_k(self, A: torch.Tensor, W: torch.Tensor, Mask: torch.Tensor,
                      residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``A [..., K]``, ``Mask [..., NG]``: packs the routing bits, then :meth:`gemm_k`."""
        lead = A.shape[:-1]
        A2 = A.reshape(-1, A.shape[-1])
        if A2.stride(-1) != 1 or A2.stride(0) % 8:
            A2 = A2.contiguous()
        M = A2.shape[0]
        NG = Mask.shape[-1]
        m8 = _mask_bytes(Mask.reshape(M, NG))
        words = (NG + 31) // 32
        row_bits = torch.empty((M, words), dtype=torch.int32, device=self.device)
        win_bits = torch.empty(((M + 127) // 128, words), dtype=torch.int32, device=self.device)
        N.check(self.lib.dpk_mask_pack(m8.data_ptr(), M, NG, row_bits.data_ptr(),
                                       win_bits.data_ptr(), _stream()))
        res2 = residual.reshape(M, self.width) if residual is not None else None
        return self.gemm_k(A2, W.contiguous(), row_bits, win_bits, NG, res2).view(*lead, self.width)
