"""Training engines behind :class:`forgeminds_b200.Trainer`.

``choose(owner, model)`` looks at the configuration, the device and the model and returns either the
:class:`~forgeminds_b200.engine.native.NativeEngine` (sm_100a kernels on a flat parameter store, any
mesh of pipeline x data x tensor parallelism) or the
:class:`~forgeminds_b200.engine.library.LibraryEngine` (``torch.distributed`` wrappers and
``torch.optim``; CPU, fp32 and the options listed in :func:`flat_store_blockers`).
"""
from __future__ import annotations

__all__ = ["choose", "flat_store_blockers"]


def flat_store_blockers(cfg, model) -> list:
    """Reasons (strings) why a run that uses the sm_100a block kernels still cannot use the flat-store engine."""
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
    if pc.ep > 1:
        why.append("expert parallelism runs on the module engine")
    return why


def choose(owner, model):
    """``FORGEMINDS_FLAT_ENGINE=1`` selects the flat-store engine even where the sm_100a kernels cannot
    run (CPU, Gloo): the blocks then run PyTorch operators, gradients are reduced with ``all_reduce``
    and the optimizer takes its PyTorch statement. The multi-process CPU tests use this to exercise
    the engine's bookkeeping (bucket hooks under pipeline schedules, skip flags, checkpoints)."""
    import os
    from .library import LibraryEngine
    forced = os.environ.get("FORGEMINDS_FLAT_ENGINE") == "1" and hasattr(model, "layers")
    if (owner.native or forced) and not owner.use_ds:
        blockers = flat_store_blockers(owner.cfg, model)
        if not blockers:
            from .native import NativeEngine
            return NativeEngine(owner, model)
        owner.engine_notes = blockers
    return LibraryEngine(owner, model)
