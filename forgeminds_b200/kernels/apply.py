"""Module surgery: route existing RMSNorm / SwiGLU modules through the fused kernels.

``patch(module)`` rewires one module instance, ``enable(model)`` walks a tree, ``revert(model)``
restores the original ``forward`` methods. Same contracts as the reference's
``forgemind/kernels/apply.py:114-223``: detection by structure and class name is conservative,
``kind=`` skips detection and validates instead, everything is idempotent, and ``split=True``
(which concatenates ``w1|w3`` into one ``gate_up`` projection and therefore renames parameters)
is never undone by ``revert``.
"""
from __future__ import annotations

import types

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["patch", "enable", "revert"]


def _norm_weight_ok(m: nn.Module) -> bool:
    w = getattr(m, "weight", None)
    return isinstance(w, nn.Parameter) and w.dim() == 1


def _looks_like_rmsnorm(m: nn.Module) -> bool:
    name = type(m).__name__.lower()
    return ("rmsnorm" in name or "rms_norm" in name) and _norm_weight_ok(m) and hasattr(m, "eps")


def _looks_like_swiglu(m: nn.Module) -> bool:
    return all(isinstance(getattr(m, n, None), nn.Linear) for n in ("w1", "w2", "w3"))


def _eps_of(m: nn.Module, x: torch.Tensor) -> float:
    eps = getattr(m, "eps", None)
    return float(torch.finfo(x.dtype).eps if eps is None else eps)     # nn.RMSNorm(eps=None) semantics


def _swap_forward(m: nn.Module, fn) -> None:
    m._fm_orig_forward = m.__dict__.get("forward")      # None: forward lives on the class
    m.forward = types.MethodType(fn, m)


def _fuse_norm(m: nn.Module) -> None:
    from . import rms_norm

    def forward(self, x):
        w = self.weight
        return rms_norm(x, w if w.dtype in (x.dtype, torch.float32) else w.to(x.dtype), _eps_of(self, x))
    _swap_forward(m, forward)


def _fuse_mlp(m: nn.Module) -> None:
    from . import swiglu

    def forward(self, x):
        return self.w2(swiglu(self.w1(x), self.w3(x)))
    _swap_forward(m, forward)


def _fuse_mlp_split(m: nn.Module) -> None:
    from . import swiglu_split
    w1, w3 = m.w1, m.w3
    if (w1.bias is None) != (w3.bias is None):
        raise ValueError("split=True needs the gate and up projections to agree on having a bias")
    fused = nn.Linear(w1.in_features, w1.out_features + w3.out_features, bias=w1.bias is not None,
                      device=w1.weight.device, dtype=w1.weight.dtype)
    with torch.no_grad():
        fused.weight.copy_(torch.cat([w1.weight, w3.weight], dim=0))
        if fused.bias is not None:
            fused.bias.copy_(torch.cat([w1.bias, w3.bias], dim=0))
    del m.w1, m.w3
    m.gate_up = fused
    m._fm_structural = True

    def forward(self, x):
        return self.w2(swiglu_split(self.gate_up(x)))
    _swap_forward(m, forward)


def patch(module: nn.Module, split: bool = False, kind: "str | None" = None) -> bool:
    """Fuse one module in place. Returns True if it was recognised (or already patched), False if
    it was left alone. ``kind="norm"`` / ``kind="mlp"`` validate the structure and raise
    ``TypeError`` when it does not fit."""
    if getattr(module, "_fm_norm", False) or getattr(module, "_fm_mlp", False):
        return True
    if kind not in (None, "norm", "mlp"):
        raise ValueError(f"kind must be 'norm', 'mlp' or None, got {kind!r}")
    if kind == "norm":
        if not _norm_weight_ok(module):
            raise TypeError(f"patch(kind='norm') needs a 1-D weight Parameter on {type(module).__name__}")
        as_norm, as_mlp = True, False
    elif kind == "mlp":
        if not _looks_like_swiglu(module):
            raise TypeError(f"patch(kind='mlp') needs Linear children w1/w2/w3 on {type(module).__name__}")
        as_norm, as_mlp = False, True
    else:
        as_norm = _looks_like_rmsnorm(module)
        as_mlp = (not as_norm) and _looks_like_swiglu(module)
    if as_norm:
        _fuse_norm(module)
        module._fm_norm = True
        return True
    if as_mlp:
        _fuse_mlp_split(module) if split else _fuse_mlp(module)
        module._fm_mlp = True
        return True
    return False


def enable(model: nn.Module, norm: bool = True, swiglu_mlp: bool = True, split: bool = False) -> nn.Module:
    """Patch every recognised norm / gated MLP under ``model``; counts land on ``model._fm_fused``."""
    counts = {"norm": 0, "mlp": 0}
    for m in list(model.modules()):
        if getattr(m, "_fm_norm", False) or getattr(m, "_fm_mlp", False):
            continue
        if norm and _looks_like_rmsnorm(m):
            patch(m)
            counts["norm"] += 1
        elif swiglu_mlp and _looks_like_swiglu(m):
            patch(m, split=split)
            counts["mlp"] += 1
    model._fm_fused = counts
    return model


def revert(module: nn.Module) -> nn.Module:
    """Give patched modules their original ``forward`` back. Structural (``split=True``) patches
    stay and are counted in ``module._fm_fused_reverted["structural"]``."""
    restored = structural = 0
    for m in module.modules():
        if getattr(m, "_fm_structural", False):
            structural += 1
            continue
        if "_fm_orig_forward" in m.__dict__:
            original = m.__dict__.pop("_fm_orig_forward")
            if original is None:
                m.__dict__.pop("forward", None)
            else:
                m.forward = original
            m.__dict__.pop("_fm_norm", None)
            m.__dict__.pop("_fm_mlp", None)
            restored += 1
    module._fm_fused_reverted = {"restored": restored, "structural": structural}
    return module
