"""On-disk layout of ``Trainer`` checkpoints and the tensor-parallel view of a state dict.

Layout (the reference's, ``forgemind/trainer.py:393-459``)::

    ckpt_dir/latest                              name of the newest step directory
    ckpt_dir/step_0000120/dcp/                   torch.distributed.checkpoint: {"model", "optim"}
    ckpt_dir/step_0000120/meta_rank{r}.json      step, epoch, batches_in_epoch, loss_ema, micro_batch
    ckpt_dir/step_0000120/offopt_rank{r}.pt      host optimizer state when the optimizer is offloaded

The fused tensor-parallel blocks keep this rank's slice of a weight as a plain tensor under the same
name on every rank; ``torch.distributed.checkpoint`` would take those for replicas and write one of
them. :func:`as_sharded` therefore presents every such tensor (and the optimizer state that belongs
to it) as a ``DTensor`` sharded over the ``tp`` mesh dimension, which is what the reference's DTensor
tensor parallelism stores, and :func:`as_local` turns a loaded state back into local tensors.
"""
from __future__ import annotations

import json
import os
import shutil

import torch


def step_dir(root: str, step: int) -> str:
    return os.path.join(root, f"step_{step:07d}")


def shard_dims(model) -> dict:
    """``{parameter name: dim}`` of the parameters that hold a tensor-parallel slice."""
    return {name: p._tp_shard_dim for name, p in model.named_parameters() if hasattr(p, "_tp_shard_dim")}


def _wrap(t, mesh, dim):
    from torch.distributed.tensor import DTensor, Shard
    if not torch.is_tensor(t) or t.dim() <= dim or hasattr(t, "to_local"):
        return t
    return DTensor.from_local(t, mesh, [Shard(dim)], run_check=False)


def as_sharded(model, msd: dict, osd, tp_mesh):
    """Replace the local slices in a (model, optimizer) state-dict pair by DTensors over ``tp_mesh``."""
    dims = shard_dims(model)
    if not dims or tp_mesh is None:
        return msd, osd
    msd = {k: (_wrap(v, tp_mesh, dims[k]) if k in dims else v) for k, v in msd.items()}

    def walk(opt_state):
        if not isinstance(opt_state, dict) or "state" not in opt_state:
            return opt_state
        state = {}
        for name, entry in opt_state["state"].items():
            if name in dims and isinstance(entry, dict):
                entry = {k: _wrap(v, tp_mesh, dims[name]) for k, v in entry.items()}
            state[name] = entry
        return {**opt_state, "state": state}

    if isinstance(osd, dict) and "state" not in osd:          # several optimizers side by side
        osd = {k: walk(v) for k, v in osd.items()}
    else:
        osd = walk(osd)
    return msd, osd


def _each_optimizer(osd, fn):
    """Apply ``fn`` to the state dict of every optimizer in ``osd`` (one, or several side by side)."""
    if isinstance(osd, dict) and "state" not in osd and "param_groups" not in osd:
        return {k: _each_optimizer(v, fn) for k, v in osd.items()}
    return fn(osd) if isinstance(osd, dict) else osd


def stage_groups(osd, stage: str, restore: bool = False):
    """Pipeline stages hold different parameters, so their ``param_groups`` differ, but a checkpoint
    stores one object per key. Keep each stage's groups under a key of its own (``param_groups@<stage>``)
    while saving / loading and put them back afterwards (``restore=True``)."""
    key = f"param_groups@{stage}"

    def move(d):
        src, dst = (key, "param_groups") if restore else ("param_groups", key)
        if src in d:
            d = dict(d)
            d[dst] = d.pop(src)
        return d
    return _each_optimizer(osd, move)


def as_local(obj):
    """Local tensors of every DTensor in a nested state."""
    if hasattr(obj, "to_local"):
        return obj.to_local()
    if isinstance(obj, dict):
        return {k: as_local(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(as_local(v) for v in obj)
    return obj


def write_meta(path: str, rank: int, meta: dict) -> None:
    with open(os.path.join(path, f"meta_rank{rank}.json"), "w") as f:
        json.dump(meta, f)


def read_meta(path: str, rank: int) -> dict:
    with open(os.path.join(path, f"meta_rank{rank}.json")) as f:
        return json.load(f)


def publish(root: str, path: str, keep_last: int) -> None:
    """Rank 0, after every rank has written: point ``latest`` at ``path`` and prune old steps."""
    with open(os.path.join(root, "latest"), "w") as f:
        f.write(os.path.basename(path))
    steps = sorted(d for d in os.listdir(root) if d.startswith("step_"))
    for old in steps[:-keep_last]:
        shutil.rmtree(os.path.join(root, old), ignore_errors=True)


def newest(root: str):
    marker = os.path.join(root, "latest")
    if not os.path.exists(marker):
        return None
    with open(marker) as f:
        return os.path.join(root, f.read().strip())
