"""Process-group bring-up, the 4-D mesh and the user-facing collectives.

One process per GPU. ``torch.distributed`` (NCCL on CUDA, Gloo on CPU) does the rendezvous,
the scalar reductions and pipeline send/recv; the bandwidth-heavy paths use the peer-memory
kernels in :mod:`forgeminds_b200.parallel.symm` on top of the groups built here.

Behaviour follows the reference's ``forgemind/distributed.py:14-187``: the same mesh axis order
``(pp, dp_replicate, dp_shard, tp)``, a flattened data-parallel group per (pp, tp) coordinate,
``ep`` groups made of consecutive data-parallel ranks and ``edp`` groups of the ranks that hold the
same expert shard.
"""
from __future__ import annotations

import datetime
import itertools
import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

from .config import ParallelConfig

_REDUCE_OPS = {"sum": "SUM", "mean": "AVG", "max": "MAX", "min": "MIN"}


@dataclass
class DistContext:
    rank: int
    world: int
    local_rank: int
    device: torch.device
    pc: ParallelConfig
    mesh: Optional[object] = None
    dp_rank: int = 0
    dp_world: int = 1
    pp_rank: int = 0
    tp_rank: int = 0
    dp_group: Optional[object] = None
    pp_group: Optional[object] = None
    tp_group: Optional[object] = None
    ep_group: Optional[object] = None
    edp_group: Optional[object] = None
    ep_rank: int = 0
    # additions: sub-groups of the data-parallel axis used by the sharded runtime
    shard_group: Optional[object] = None       # dp_shard axis
    replicate_group: Optional[object] = None   # dp_replicate axis
    shard_rank: int = 0
    replicate_rank: int = 0
    dp_ranks: list = field(default_factory=list)

    @property
    def is_main(self) -> bool:
        return self.rank == 0

    @property
    def device_type(self) -> str:
        return self.device.type

    def barrier(self) -> None:
        if self.world > 1:
            dist.barrier()

    # The helpers below hand back device tensors; no value is read on the host.
    def _reduced(self, x, group, op=None):
        y = x.clone()
        dist.all_reduce(y, group=group) if op is None else dist.all_reduce(y, op=op, group=group)
        return y

    def sum_over_dp(self, x: torch.Tensor) -> torch.Tensor:
        if self.dp_world <= 1 or self.dp_group is None:
            return x
        return self._reduced(x, self.dp_group)

    def mean_over_dp(self, x: torch.Tensor) -> torch.Tensor:
        if self.dp_world <= 1 or self.dp_group is None:
            return x
        return self._reduced(x, self.dp_group).div_(self.dp_world)

    def sum_over_pp(self, x: torch.Tensor) -> torch.Tensor:
        if self.pc.pp <= 1 or self.world <= 1 or self.pp_group is None:
            return x
        return self._reduced(x, self.pp_group)

    def all_min_int(self, x: torch.Tensor) -> torch.Tensor:
        """World-wide MIN of a 0/1 flag: the result is 1 only if every rank voted 1."""
        if self.world <= 1:
            return x
        return self._reduced(x, None, dist.ReduceOp.MIN)


def log(ctx: Optional[DistContext], *args, **kwargs) -> None:
    if ctx is None or ctx.rank == 0:
        print(*args, flush=True, **kwargs)


# ------------------------------------------------------------------------------ user collectives
def _multi() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def all_reduce(tensor: torch.Tensor, reduce_op: str = "mean") -> torch.Tensor:
    """In-place reduction over the world (``mean | sum | max | min``). With one process the very
    same tensor object is returned and no collective runs; an unknown ``reduce_op`` raises
    ``KeyError`` in either case (reference ``forgemind/distributed.py:85-92``)."""
    op_name = _REDUCE_OPS[reduce_op]
    if not _multi():
        return tensor
    dist.all_reduce(tensor, op=getattr(dist.ReduceOp, op_name))
    return tensor


def broadcast(tensor: torch.Tensor, src: int = 0) -> torch.Tensor:
    if _multi():
        dist.broadcast(tensor, src=src)
    return tensor


def all_gather(tensor: torch.Tensor) -> torch.Tensor:
    """Concatenate every rank's tensor along dim 0."""
    if not _multi():
        return tensor
    world = dist.get_world_size()
    out = tensor.new_empty((world * tensor.shape[0],) + tuple(tensor.shape[1:])) if tensor.dim() else \
        tensor.new_empty((world,))
    if tensor.dim() == 0:
        parts = [torch.empty_like(tensor) for _ in range(world)]
        dist.all_gather(parts, tensor)
        return torch.cat([p.reshape(1) for p in parts], 0)
    dist.all_gather_into_tensor(out, tensor.contiguous())
    return out


def barrier() -> None:
    if _multi():
        dist.barrier()


# ------------------------------------------------------------------------------ bring-up
def _coords(pc: ParallelConfig, rank: int):
    """(pp, dp_replicate, dp_shard, tp) coordinate of a global rank in row-major mesh order."""
    t = rank % pc.tp
    rest = rank // pc.tp
    s = rest % pc.dp_shard
    rest //= pc.dp_shard
    r = rest % pc.dp_replicate
    p = rest // pc.dp_replicate
    return p, r, s, t


def _rank_of(pc: ParallelConfig, p: int, r: int, s: int, t: int) -> int:
    return ((p * pc.dp_replicate + r) * pc.dp_shard + s) * pc.tp + t


def init_distributed(pc: ParallelConfig, backend: Optional[str] = None) -> DistContext:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    on_gpu = torch.cuda.is_available()
    if on_gpu:
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")

    if world > 1 and not dist.is_initialized():
        dist.init_process_group(backend or ("nccl" if on_gpu else "gloo"), rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=pc.init_timeout_s),
                                device_id=device if on_gpu else None)

    outer = pc.pp * pc.tp * pc.dp_replicate
    if pc.dp_shard == -1:
        assert world % outer == 0, f"world {world} not divisible by pp*tp*dp_replicate={outer}"
        pc.dp_shard = world // outer
    product = pc.pp * pc.dp_replicate * pc.dp_shard * pc.tp
    assert product == world, f"pp*dp_replicate*dp_shard*tp = {product} != world {world}"
    dp_world = pc.dp_replicate * pc.dp_shard
    assert dp_world % pc.ep == 0, f"ep={pc.ep} must divide dp world {dp_world}"

    ctx = DistContext(rank, world, local, device, pc, dp_world=dp_world)
    if world == 1:
        return ctx

    from torch.distributed.device_mesh import init_device_mesh
    ctx.mesh = init_device_mesh(device.type, (pc.pp, pc.dp_replicate, pc.dp_shard, pc.tp),
                                mesh_dim_names=("pp", "dp_replicate", "dp_shard", "tp"))
    p, r, s, t = _coords(pc, rank)
    ctx.pp_rank, ctx.tp_rank = p, t
    ctx.replicate_rank, ctx.shard_rank = r, s
    ctx.dp_rank = r * pc.dp_shard + s
    ctx.pp_group = ctx.mesh["pp"].get_group()
    ctx.tp_group = ctx.mesh["tp"].get_group()
    ctx.shard_group = ctx.mesh["dp_shard"].get_group()
    ctx.replicate_group = ctx.mesh["dp_replicate"].get_group()

    # Every rank walks the same loops so that new_group is called in the same order everywhere.
    for pi, ti in itertools.product(range(pc.pp), range(pc.tp)):
        members = [_rank_of(pc, pi, ri, si, ti)
                   for ri in range(pc.dp_replicate) for si in range(pc.dp_shard)]
        g = dist.new_group(members)
        mine = rank in members
        if mine:
            ctx.dp_group, ctx.dp_ranks = g, members
        if pc.ep == 1:
            continue
        teams = [members[i:i + pc.ep] for i in range(0, len(members), pc.ep)]
        for team in teams:
            g = dist.new_group(team)
            if rank in team:
                ctx.ep_group, ctx.ep_rank = g, team.index(rank)
        for slot in range(pc.ep):
            peers = [team[slot] for team in teams]
            g = dist.new_group(peers)
            if rank in peers:
                ctx.edp_group = g
    return ctx


def cleanup() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
