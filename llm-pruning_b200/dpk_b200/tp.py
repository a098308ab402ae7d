"""Tensor-parallel partitioning of the routed layer (host-side logic).

The routed FFN shards by channel groups and routed attention by KV-head groups, the
Megatron-style plan the reference sketches for its wrappers (gate/up/q/k/v column
parallel, down/o row parallel, ``WIDE/transformer_fsdp_hook.py:44-54``; disabled there
with ``tensor_parallel_size=1``, ``WIDE/mainloop.py:602``).  Inputs and routers are
replicated, so every rank derives the same mask and slices its own columns; the only
exchange is the sum of the partial outputs of the row-parallel projection.

Everything here is plain ``torch`` / ``torch.distributed`` and runs on CPU ranks
(``gloo``) as well as GPU ranks (``nccl``); the per-rank compute is injected.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def group_range(num_groups: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous block of routed groups owned by ``rank``."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if num_groups % world:
        raise ValueError(f"{num_groups} groups do not split evenly over {world} ranks")
    per = num_groups // world
    return rank * per, (rank + 1) * per


def shard_ffn_weights(gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, num_groups: int,
                      world: int, rank: int):
    """Rows of ``gate``/``up`` ``[I,H]`` and columns of ``down`` ``[H,I]`` of this rank's
    groups (contiguous copies)."""
    inter = gate.shape[0]
    if inter % num_groups:
        raise ValueError(f"I={inter} is not divisible by {num_groups} groups")
    width = inter // num_groups
    g0, g1 = group_range(num_groups, world, rank)
    c0, c1 = g0 * width, g1 * width
    return gate[c0:c1].contiguous(), up[c0:c1].contiguous(), down[:, c0:c1].contiguous()


def shard_mask(mask: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """This rank's group columns of a replicated ``[..., NG]`` routing mask."""
    g0, g1 = group_range(mask.shape[-1], world, rank)
    return mask[..., g0:g1]


def shard_attention(q_weight: torch.Tensor, k_weight: torch.Tensor, v_weight: torch.Tensor,
                    o_weight: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int,
                    world: int, rank: int):
    """KV-head-group sharding: rank owns ``Hk/world`` KV heads with their ``Hq/Hk`` query
    heads -- rows of ``q/k/v`` weights, columns of the ``o`` weight."""
    k0, k1 = group_range(num_kv_heads, world, rank)
    rep = num_q_heads // num_kv_heads
    q0, q1 = k0 * rep * head_dim, k1 * rep * head_dim
    kv0, kv1 = k0 * head_dim, k1 * head_dim
    return (q_weight[q0:q1].contiguous(), k_weight[kv0:kv1].contiguous(),
            v_weight[kv0:kv1].contiguous(), o_weight[:, q0:q1].contiguous())


class TensorParallelFFN:
    """Row-parallel sum around a per-rank routed FFN.

    ``local_ffn(x, local_mask) -> partial_y`` computes this rank's groups (on a GPU rank:
    a :class:`dpk_b200.ffn.RoutedFFN` built from :func:`shard_ffn_weights`).  The call
    slices the replicated mask, runs the local part and all-reduces the partial outputs
    in place.  ``chunks > 1`` splits the tokens so that the all-reduce of one chunk can
    overlap the compute of the next when ``comm_stream`` is given (GPU ranks).
    """

    def __init__(self, local_ffn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                 num_groups: int, process_group: Optional[dist.ProcessGroup] = None):
        self.local_ffn = local_ffn
        self.num_groups = num_groups
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        group_range(num_groups, self.world, self.rank)     # validates divisibility early

    def __call__(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        if mask.shape[-1] != self.num_groups:
            raise ValueError(f"Mask has {mask.shape[-1]} groups, expected {self.num_groups}")
        y = self.local_ffn(x, shard_mask(mask, self.world, self.rank))
        if self.world > 1:
            dist.all_reduce(y, group=self.pg)
        return y


def owner_block_sum(partial: torch.Tensor, process_group: Optional[dist.ProcessGroup] = None,
                    residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The data movement of the fused row-parallel sum (:mod:`dpk_b200.peer`) written with plain
    point-to-point messages, for ranks that cannot map each other's memory (other nodes, CPU
    ranks): rows are owned in contiguous blocks of whole 128-token windows
    (:func:`dpk_b200.peer.rows_per_owner`); every rank sends each owner its partial rows of that
    owner's block, the owner adds the ``world`` contributions in rank order (fp32, plus the
    residual rows when given), rounds once and sends the finished rows to everyone.
    ``partial``: ``[M, N]``.  Returns the summed ``[M, N]`` (same on every rank, bit for bit)."""
    from .peer import rows_per_owner
    world = dist.get_world_size(process_group) if dist.is_initialized() else 1
    rank = dist.get_rank(process_group) if dist.is_initialized() else 0
    M, N = partial.shape
    R = rows_per_owner(M, world)
    block = lambda o: slice(min(o * R, M), min((o + 1) * R, M))
    mine = block(rank)
    # first half: partial rows to their owners
    got = [None] * world
    reqs = []
    for o in range(world):
        if o == rank or block(o).start == block(o).stop:
            continue
        reqs.append(dist.isend(partial[block(o)].contiguous(), o, group=process_group))
    for src in range(world):
        if src == rank or mine.start == mine.stop:
            continue
        got[src] = torch.empty_like(partial[mine])
        reqs.append(dist.irecv(got[src], src, group=process_group))
    for r in reqs:
        r.wait()
    got[rank] = partial[mine]
    out = torch.empty_like(partial)
    if mine.start != mine.stop:
        acc = torch.zeros(partial[mine].shape, dtype=torch.float32, device=partial.device)
        for src in range(world):                       # rank order: the same sum on every owner
            acc += got[src].to(torch.float32)
        if residual is not None:
            acc += residual[mine].to(torch.float32)
        out[mine] = acc.to(partial.dtype)
    # second half: finished rows to everyone
    reqs = []
    for dst in range(world):
        if dst != rank and mine.start != mine.stop:
            reqs.append(dist.isend(out[mine].contiguous(), dst, group=process_group))
    bufs = {}
    for o in range(world):
        if o != rank and block(o).start != block(o).stop:
            bufs[o] = torch.empty_like(out[block(o)])
            reqs.append(dist.irecv(bufs[o], o, group=process_group))
    for r in reqs:
        r.wait()
    for o, buf in bufs.items():
        out[block(o)] = buf
    return out
