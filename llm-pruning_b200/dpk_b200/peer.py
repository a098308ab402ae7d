"""Row-parallel sum fused into the reduction-width projection (tensor-parallel ranks).

Under the split the reference sketches for its wrappers (down / o projections row
parallel, ``WIDE/transformer_fsdp_hook.py:44-54``) every rank ends a sub-block with a
partial ``[M,N]`` sum that has to be added over the ranks.  Instead of writing the partial
sums to local memory and handing them to an all-reduce, the projection kernel stores each
128-token window straight into the memory of the rank that owns those rows while the other
tiles are still being computed; each owner then adds the slabs it received (fp32, optional
residual) and stores the finished rows into every rank's output.  Between the two kernels,
and after the second, the ranks meet at a barrier ordered on the stream: a one-element NCCL
all-reduce (``barrier_mode = "nccl"``, the default) or ``dpk_peer_barrier``, one small kernel
per rank that publishes an arrival flag in every peer's memory and waits, with a time limit,
for the peers' flags (``barrier_mode = "flags"``; same results, but measured slower and less
steady than the NCCL barrier on two GPUs -- 12.9-14.3 against 11.5-11.7 ms per step of the
70B-shaped layer -- so it is not the default).

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
FLAG_BYTES = 256            # arrival slots of the flag barrier, at the end of the peer buffer


def rows_per_owner(M: int, world: int) -> int:
    """Token rows each rank owns: an equal share rounded up to whole 128-token windows."""
    if world < 1 or world > MAX_WORLD:
        raise ValueError(f"world must be 1..{MAX_WORLD}")
    share = (max(M, 1) + world - 1) // world
    return (share + WINDOW - 1) // WINDOW * WINDOW


def owner_of_row(row: int, M: int, world: int) -> int:
    return row // rows_per_owner(M, world)


def half_split(M: int, world: int, width: int, part: Optional[int]):
    """``(row0, rows, staging offset in elements)`` of the whole call (``part`` None) or of its
    first / second half (0 / 1).  The first half ends on a window boundary; each half is its own
    ownership split, and the second half's slabs start where the first half's end."""
    if part is None:
        return 0, M, 0
    M0 = min(M, ((M + 1) // 2 + WINDOW - 1) // WINDOW * WINDOW)
    if part == 0:
        return 0, M0, 0
    return M0, M - M0, world * rows_per_owner(M0, world) * width


def staging_rows(max_rows: int, world: int) -> int:
    """Rows per slab a staging buffer is sized for: the share of ``max_rows`` plus two windows,
    which covers the separate rounding of the two halves."""
    return rows_per_owner(max_rows, world) + 2 * WINDOW


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

    barrier_mode = "nccl"        # or "flags": see the module docstring
    barrier_timeout_ms = 2000    # flag barrier: how long a rank waits for its peers

    def __init__(self, world: int, rank: int, max_rows: int, width: int, dtype: torch.dtype,
                 device: torch.device, stage: torch.Tensor, out: torch.Tensor,
                 stage_ptrs: Sequence[int], out_ptrs: Sequence[int],
                 barrier: Callable[[], None], keep=(), flag_ptrs: Sequence[int] = ()):
        self.world, self.rank, self.max_rows, self.width = world, rank, max_rows, width
        self.dtype, self.device = dtype, device
        self.stage, self.out = stage, out
        self._stage_ptrs, self._out_ptrs = list(stage_ptrs), list(out_ptrs)
        self._nccl_barrier = barrier
        self._flag_ptrs = list(flag_ptrs)       # every rank's arrival slots (peer-mapped), or empty
        self._epoch = 0
        self.halves = 1          # 2: split the tokens; the second half's projection hides the first half's gather
        self._side = None
        self._keep = keep
        self.lib = N.load()
        self.code = 1 if dtype == torch.bfloat16 else 0
        self._ws = None
        self.timers = None      # dict -> lists of CUDA events at the five points of a fused sum

    def _barrier(self) -> None:
        """All ranks have finished what they enqueued before this point (stream-ordered)."""
        if self.barrier_mode == "flags" and self._flag_ptrs:
            self._epoch += 1
            N.check(self.lib.dpk_peer_barrier(_ptr_table(self._flag_ptrs), self._flag_ptrs[self.rank],
                                              self.world, self.rank, self._epoch,
                                              int(self.barrier_timeout_ms), _stream()))
        else:
            self._nccl_barrier()

    # ---- construction -----------------------------------------------------------------
    @staticmethod
    def _sizes(world: int, max_rows: int, width: int):
        R = staging_rows(max_rows, world)
        return R, world * R * width * 2

    @classmethod
    def connect(cls, max_rows: int, width: int, dtype: torch.dtype, device: torch.device,
                group: Optional[dist.ProcessGroup] = None) -> "RowParallelSum":
        """Collective over ``group``: allocate this rank's buffers, exchange the IPC
        handles, map the peers'."""
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        _, nbytes = cls._sizes(world, max_rows, width)
        lib = N.load()
        # Every rank takes part in every exchange below even when something failed locally, so
        # that a failure on one rank becomes the same exception on all of them instead of a
        # rank waiting in a collective the others never enter.
        problem = None
        with torch.cuda.device(device):
            base = C.c_void_p()
            handle = C.create_string_buffer(64)
            try:
                N.check(lib.dpk_peer_alloc(2 * nbytes + FLAG_BYTES, C.byref(base), handle))
            except Exception as exc:          # noqa: BLE001 - reported to all ranks below
                problem = f"rank {rank}: {exc}"
            handles: List[Optional[bytes]] = [None] * world
            dist.all_gather_object(handles, None if problem else handle.raw, group=group)
            bases = []
            if all(h is not None for h in handles):
                for r in range(world):
                    if r == rank:
                        bases.append(base.value)
                        continue
                    p = C.c_void_p()
                    try:
                        N.check(lib.dpk_peer_open(handles[r], C.byref(p)))
                        bases.append(p.value)
                    except Exception as exc:  # noqa: BLE001
                        problem = problem or f"rank {rank} mapping rank {r}: {exc}"
                        break
            elif problem is None:
                problem = "a peer could not allocate its buffer"
            problems: List[Optional[str]] = [None] * world
            dist.all_gather_object(problems, problem, group=group)
            if any(problems):
                for q in bases:
                    if q != base.value:
                        lib.dpk_peer_close(q)
                if base.value:
                    lib.dpk_peer_free(base)
                raise RuntimeError("peer buffers unavailable: " + "; ".join(x for x in problems if x))
            raw = torch.as_tensor(_DeviceBytes(base.value, 2 * nbytes + FLAG_BYTES), device=device)
        stage = raw[:nbytes].view(dtype)
        out = raw[nbytes:2 * nbytes].view(dtype)
        raw[2 * nbytes:].zero_()                 # arrival slots start at zero on every rank ...
        torch.cuda.synchronize(device)
        dist.barrier(group=group)                # ... before any rank can publish into them
        token = torch.zeros(1, device=device)

        def barrier():
            dist.all_reduce(token, group=group)

        self = cls(world, rank, max_rows, width, dtype, device, stage, out, bases,
                   [b + nbytes for b in bases], barrier, keep=(raw, token),
                   flag_ptrs=[b + 2 * nbytes for b in bases])
        self._mapped = [b for r, b in enumerate(bases) if r != rank]
        self._owned = base.value
        return self

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's.  Collective in effect: call it on every
        rank, after the last use, with the stream idle."""
        torch.cuda.synchronize(self.device)
        for q in getattr(self, "_mapped", []):
            self.lib.dpk_peer_close(q)
        if getattr(self, "_owned", None):
            self.lib.dpk_peer_free(self._owned)
        self._mapped, self._owned = [], None
        self.stage = self.out = None
        self._keep = ()

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

    # ---- the two kernels ------------------------------------------------------------------
    def _part(self, M: int, part: Optional[int]):
        return half_split(M, self.world, self.width, part)

    def scatter(self, A2: torch.Tensor, W: torch.Tensor, row_bits: torch.Tensor,
                win_bits: torch.Tensor, NG: int, part: Optional[int] = None) -> None:
        """Projection kernel: this rank's partial sums go to the owners' staging buffers
        (``part``: ``None`` = all rows, 0 / 1 = first / second half of the tokens)."""
        M, K = A2.shape
        if M > self.max_rows or W.shape != (self.width, K):
            raise ValueError("shape outside what this RowParallelSum was built for")
        row0, rows, soff = self._part(M, part)
        if rows <= 0:
            return
        R = rows_per_owner(rows, self.world)
        need = self.lib.dpk_gemm_k_scatter_workspace_bytes(rows, self.width, self.width)
        if need and (self._ws is None or self._ws.numel() < need):
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        esz = A2.element_size()
        words = row_bits.shape[1]
        stage_tab = _ptr_table([b + soff * 2 for b in self._stage_ptrs])
        N.check(self.lib.dpk_gemm_k_scatter(
            A2.data_ptr() + row0 * A2.stride(0) * esz, A2.stride(0), W.data_ptr(), W.stride(0),
            row_bits.data_ptr() + row0 * words * 4, win_bits.data_ptr() + (row0 // WINDOW) * words * 4,
            stage_tab, self.world, self.rank, R, self.width, rows, self.width, K, NG, self.code,
            self._ws.data_ptr() if need else None, need, _stream()))

    def reduce(self, M: int, residual: Optional[torch.Tensor] = None, part: Optional[int] = None,
               max_blocks: int = 0) -> torch.Tensor:
        """Reduce + gather kernel: sum the received slabs of the rows this rank owns and store
        them into every rank's output."""
        if residual is not None and (residual.shape != (M, self.width) or not residual.is_contiguous()):
            raise ValueError("residual must be a contiguous [M, width] tensor")
        row0, rows, soff = self._part(M, part)
        if rows > 0:
            R = rows_per_owner(rows, self.world)
            ooff = row0 * self.width * 2
            out_tab = _ptr_table([b + ooff for b in self._out_ptrs])
            N.check(self.lib.dpk_reduce_gather(
                self.stage.data_ptr() + soff * 2, out_tab,
                residual.data_ptr() + ooff if residual is not None else None, self.world, self.rank, R,
                rows, self.width, self.width, self.code, max_blocks, _stream()))
        return self.out[:M * self.width].view(M, self.width)

    def gemm_k(self, A2: torch.Tensor, W: torch.Tensor, row_bits: torch.Tensor,
               win_bits: torch.Tensor, NG: int, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        M = A2.shape[0]
        if self.halves == 2 and M >= 4 * WINDOW * self.world:
            return self._gemm_k_halves(A2, W, row_bits, win_bits, NG, residual)
        self._mark("start")
        self.scatter(A2, W, row_bits, win_bits, NG)
        self._mark("scatter")
        self._barrier()          # every rank's partial sums have landed
        self._mark("barrier1")
        y = self.reduce(M, residual)
        self._mark("reduce")
        self._barrier()          # every owner's rows have landed; staging may be reused
        self._mark("barrier2")
        return y

    def _gemm_k_halves(self, A2, W, row_bits, win_bits, NG, residual):
        """The tokens in two halves: while the second half is being projected (tensor cores,
        stores of partial sums), the first half is reduced and gathered on a second stream
        (loads from local memory, stores over the links) by a grid small enough to share the
        SMs with the projection."""
        M = A2.shape[0]
        main = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        self.scatter(A2, W, row_bits, win_bits, NG, part=0)
        self._barrier()
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            self.reduce(M, residual, part=0, max_blocks=148)
        self.scatter(A2, W, row_bits, win_bits, NG, part=1)
        self._barrier()
        y = self.reduce(M, residual, part=1)
        main.wait_stream(self._side)
        self._barrier()
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
