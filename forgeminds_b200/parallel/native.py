"""Data / tensor / expert parallel wrappers.

Two implementations live behind each entry point:

* the **library baseline** -- ``torch.distributed`` FSDP2 (``fully_shard``), ``DistributedDataParallel``
  and DTensor tensor parallelism, exactly what the reference wires up in
  ``forgemind/parallel/native.py:21-113``. It is what runs on CPU/Gloo and what the fused paths are
  measured against;
* the **sm_100a engine** (:mod:`forgeminds_b200.engine.native` with :mod:`forgeminds_b200.parallel.flat`,
  ``.peer`` and ``.tp``): a flat fp32 master store with bf16 working weights, gradient reduction,
  clipping and AdamW in peer-memory kernels, tensor parallelism fused with its collectives. The
  trainer selects it; the functions here are what everything else runs on.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..distributed import DistContext

__all__ = ["has_moe", "apply_tp", "apply_fsdp", "apply_ddp", "sync_expert_grads", "expert_params"]


def has_moe(model) -> bool:
    return any(getattr(b, "is_moe", False) for b in model.layers.values())


def expert_params(model) -> list:
    """Parameters that belong to (rank-local) experts; cached by the trainer."""
    return [p for n, p in model.named_parameters() if ".experts." in n]


# ------------------------------------------------------------------------------ tensor parallel
def apply_tp(model, ctx: DistContext, plan=None):
    """Column-parallel ``wq/wk/wv/w1/w3`` and row-parallel ``wo/w2`` inside every block.

    GPU + bf16 models get the fused implementation (all-gather -> GEMM and GEMM -> reduce-scatter
    over peer memory, see :mod:`forgeminds_b200.parallel.tp`); otherwise DTensor
    ``parallelize_module`` is used.
    """
    cfg = model.cfg
    tp = ctx.pc.tp
    assert cfg.n_heads % tp == 0 and cfg.n_kv_heads % tp == 0, "heads must divide tp"
    plan = plan or model.tp_plan()
    if ctx.device.type == "cuda" and getattr(cfg, "native", None) is not False:
        from . import tp as fused_tp
        if fused_tp.usable(ctx):
            return fused_tp.shard_model(model, ctx, plan)
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module
    style = {"col": ColwiseParallel, "row": RowwiseParallel}
    mesh = ctx.mesh["tp"]
    hits = 0
    for blk in model.layers.values():
        present = {name for name, _ in blk.named_modules()}
        sub = {name: style[kind]() for name, kind in plan.items() if name in present}
        if sub:
            parallelize_module(blk, mesh, sub)
            hits += len(sub)
    if not hits:
        raise RuntimeError("apply_tp: no module matched the tensor-parallel plan")
    model._fm_tp = "dtensor"
    # DTensor parameters go through PyTorch operators: the kernel path of the blocks takes plain tensors only
    for blk in model.layers.values():
        if hasattr(blk, "native"):
            blk.native = False
    return model


# ------------------------------------------------------------------------------ sharded / replicated data parallel
def _dp_mesh(ctx: DistContext):
    pc = ctx.pc
    dims = tuple(n for n, size in (("dp_replicate", pc.dp_replicate), ("dp_shard", pc.dp_shard)) if size > 1)
    if not dims:
        raise ValueError("apply_fsdp called with no shard/replicate dimension")
    return ctx.mesh[dims] if len(dims) > 1 else ctx.mesh[dims[0]]


def apply_fsdp(model, ctx: DistContext, bf16=True, cpu_offload=False, reshard=True):
    """FSDP2 / HSDP: per-block sharding then the root; bf16 parameters for compute, fp32 gradient
    reduction; the last block and the root never reshard after forward."""
    pc = ctx.pc
    if pc.ep > 1:
        raise NotImplementedError("expert parallelism + sharded data parallelism needs a separate expert mesh; "
                                  "use dp_replicate with ep")
    from torch.distributed.fsdp import CPUOffloadPolicy, MixedPrecisionPolicy, fully_shard
    kw = dict(mesh=_dp_mesh(ctx))
    if bf16:
        kw["mp_policy"] = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    if cpu_offload:
        kw["offload_policy"] = CPUOffloadPolicy()
    blocks = list(model.layers.values())
    for i, blk in enumerate(blocks):
        fully_shard(blk, reshard_after_forward=bool(reshard) and i < len(blocks) - 1, **kw)
    fully_shard(model, reshard_after_forward=False if blocks else reshard, **kw)
    return model


def apply_ddp(model, ctx: DistContext):
    """``DistributedDataParallel`` over the flattened data-parallel group; rank-local experts are
    kept out of the reducer when expert parallelism is on. Buffers are not re-broadcast at every
    forward: the only buffers of the models here are RoPE tables, which every rank computes itself, and
    an in-place broadcast would invalidate the graphs of the micro-batches a pipeline schedule keeps
    in flight."""
    from torch.nn.parallel import DistributedDataParallel as DDP
    if ctx.pc.ep > 1:
        skip = [n for n, _ in model.named_parameters() if ".experts." in n]
        DDP._set_params_and_buffers_to_ignore_for_model(model, skip)
    unused = has_moe(model) and ctx.pc.ep == 1 and not ctx.pc.ddp_static_graph
    return DDP(model, device_ids=[ctx.local_rank] if ctx.device.type == "cuda" else None,
               process_group=ctx.dp_group, gradient_as_bucket_view=True, broadcast_buffers=False,
               static_graph=ctx.pc.ddp_static_graph, find_unused_parameters=unused)


def sync_expert_grads(model, ctx: DistContext, params=None) -> None:
    """Finish the gradients of rank-local experts: they already hold the sum over the tokens of the
    ep group (all-to-all backward); add the other replicas of the same shard (``edp`` group) and
    divide by the data-parallel world so they are scaled like every other gradient."""
    if ctx.pc.ep == 1 or ctx.world == 1:
        return
    grads = [p.grad for p in (expert_params(model) if params is None else params) if p.grad is not None]
    if not grads:
        return
    if ctx.edp_group is not None and dist.get_world_size(ctx.edp_group) > 1:
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, group=ctx.edp_group)
        torch._foreach_copy_(grads, [t.view_as(g) for t, g in zip(flat.split([g.numel() for g in grads]), grads)])
    torch._foreach_div_(grads, ctx.dp_world)
