"""Activation checkpointing per transformer block: ``full`` recomputes the whole block in the
backward, ``selective`` keeps matmul / attention outputs and recomputes the cheap rest.

Interface of the reference's ``forgemind/parallel/ac.py:22-48``. The selective save-list names the
aten matmul and SDPA ops for the PyTorch path. Blocks that run on the sm_100a kernels implement the
same policy inside their autograd functions: they keep the residual stream, the projection and
attention outputs and the per-row statistics, and recompute the normalised activations and the
SwiGLU product in the backward; with ``selective`` they are therefore left unwrapped.
"""
from __future__ import annotations

import functools

import torch
from torch.utils.checkpoint import CheckpointPolicy, checkpoint, create_selective_checkpoint_contexts

_KEEP_NAMES = ("mm", "addmm", "bmm", "baddbmm", "_scaled_dot_product_flash_attention",
               "_scaled_dot_product_efficient_attention", "_scaled_dot_product_cudnn_attention",
               "_scaled_dot_product_flash_attention_for_cpu")
_KEEP = {getattr(torch.ops.aten, n).default for n in _KEEP_NAMES if hasattr(torch.ops.aten, n)}


def _selective_policy(ctx, op, *args, **kwargs):
    return CheckpointPolicy.MUST_SAVE if op in _KEEP else CheckpointPolicy.PREFER_RECOMPUTE


def apply_activation_checkpointing(model, mode: str = "full", preserve_rng_state: bool = False):
    """Patch ``block.forward`` of every entry of ``model.layers`` in place (module names unchanged)."""
    if mode == "none":
        return model
    if mode not in ("full", "selective"):
        raise ValueError(f"ac must be none|full|selective, got {mode!r}")
    options = dict(use_reentrant=False, preserve_rng_state=preserve_rng_state)
    if mode == "selective":
        options["context_fn"] = functools.partial(create_selective_checkpoint_contexts, _selective_policy)
    for blk in model.layers.values():
        if getattr(blk, "_fm_ac", False):
            continue
        plain = blk.forward

        def guarded(*args, _plain=plain, _blk=blk, _opts=options, **kwargs):
            if mode == "selective" and args and _runs_native(_blk, args[0]):
                return _plain(*args, **kwargs)
            return checkpoint(_plain, *args, **kwargs, **_opts)
        blk.forward = guarded
        blk._fm_ac = mode
    return model


def _runs_native(blk, x) -> bool:
    if not (torch.is_tensor(x) and x.is_cuda):
        return False
    from ..models.gpt import _native_ok
    return hasattr(blk, "_forward_native") and _native_ok(x, getattr(blk, "native", None))
