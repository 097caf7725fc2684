"""Training engines behind :class:`forgeminds_b200.Trainer`.

``choose(owner, model)`` looks at the configuration, the device and the model and returns either the
:class:`~forgeminds_b200.engine.native.NativeEngine` (sm_100a kernels on a flat parameter store, any
mesh of pipeline x data x tensor parallelism) or the
:class:`~forgeminds_b200.engine.library.LibraryEngine` (``torch.distributed`` wrappers and
``torch.optim``; CPU, fp32 and the options listed in :func:`flat_store_blockers`).
"""
from __future__ import annotations

__all__ = ["choose", "flat_store_blockers"]


def flat_store_blockers(cfg, model, kernels: bool = True) -> list:
    """Reasons (strings) why a run cannot use the flat-store engine. ``kernels``: the blocks run on the
    sm_100a kernels (false only when the engine is forced on for CPU tests)."""
    tc, pc, oc, qc = cfg.train, cfg.parallel, cfg.offload, cfg.quant
    why = []
    if oc.optimizer:
        why.append("offload.optimizer keeps the optimizer state on the host")
    if qc.optimizer_8bit:
        why.append("quant.optimizer_8bit uses a third-party optimizer")
    if pc.fsdp_cpu_offload:
        why.append("parallel.fsdp_cpu_offload is an FSDP2 policy")
    if tc.compile:
        why.append("train.compile wraps the blocks")
    if qc.mode not in ("none", "fp8", "int8"):
        why.append(f"quant.mode={qc.mode!r} freezes the base weights")
    if pc.tp > 1 and isinstance(getattr(model, "_fm_tp", None), str):
        why.append("tensor parallelism fell back to DTensor")
    if pc.ep > 1 and kernels and getattr(model, "_fm_ep", None) is None:
        why.append("expert parallelism without the fused dispatch / combine kernels (parallel.fused_comm off, "
                   "more than 8 ranks per group, or experts offloaded)")
    if pc.ep > 1 and oc.experts:
        why.append("offload.experts keeps the experts in host memory")
    return why


def resident_bytes(model, cfg, ctx) -> int:
    """Device memory the flat-store engine needs for this rank's slice of the model: bf16 working weights
    (2 bytes per parameter), fp32 gradients (4) and fp32 masters (4) whole, AdamW moments (8) divided by
    the number of ranks that share the optimizer state."""
    n = sum(p.numel() for p in model.parameters() if p.requires_grad)
    pc = cfg.parallel
    share = max(1, ctx.dp_world if pc.dp_shard <= 1 else pc.dp_shard) if pc.fused_comm else 1
    return int(n * (10 + 8 / share))


def choose(owner, model):
    """``FORGEMINDS_FLAT_ENGINE=1`` selects the flat-store engine even where the sm_100a kernels cannot
    run (CPU, Gloo): the blocks then run PyTorch operators, gradients are reduced with ``all_reduce``
    and the optimizer takes its PyTorch statement. The multi-process CPU tests use this to exercise
    the engine's bookkeeping (bucket hooks under pipeline schedules, skip flags, checkpoints).
    ``FORGEMINDS_FLAT_ENGINE=0`` keeps a run on the library engine (blocks still on the kernels), which is
    how the GPU tests obtain the trajectory to compare with."""
    import os
    from .library import LibraryEngine
    switch = os.environ.get("FORGEMINDS_FLAT_ENGINE", "")
    forced = switch == "1" and hasattr(model, "layers")
    if (owner.native or forced) and not owner.use_ds and switch != "0":
        blockers = flat_store_blockers(owner.cfg, model, kernels=bool(owner.native))
        if owner.native and owner.ctx.device.type == "cuda" and owner.ctx.dp_world > 1 and not blockers:
            import torch
            budget = int(owner.cfg.parallel.fsdp_resident_bytes) or \
                int(0.8 * torch.cuda.get_device_properties(owner.ctx.device).total_memory)
            need = resident_bytes(model, owner.cfg, owner.ctx)
            if need > budget:
                blockers.append(f"the flat store would need {need / 2 ** 30:.0f} GiB per GPU for weights, gradients and "
                                f"optimizer state (budget {budget / 2 ** 30:.0f} GiB): parameters must be sharded")
        if not blockers:
            from .native import NativeEngine
            return NativeEngine(owner, model)
        owner.engine_notes = blockers
    return LibraryEngine(owner, model)
