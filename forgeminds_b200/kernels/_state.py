"""Backend switch and path statistics shared by the kernel wrappers.

``set_backend("auto" | "fallback" | "native")`` -- ``"fallback"`` forces the PyTorch statements
even on a GPU (for A/B runs), ``"native"`` insists on the CUDA kernels and raises where they cannot
run. ``"triton"`` is accepted as an alias of ``"native"`` for scripts written against the
reference (``forgemind/kernels/_common.py:44-111``); no Triton code exists in this library.
"""
from __future__ import annotations

import torch

HAS_TRITON = False           # kept for API parity: the kernels here are CUDA, not Triton
_BACKEND = "auto"
_COUNTS = {"fast": 0, "fallback": 0, "reason": {}}
_FORCE_CUSTOM_OPS = False
_DTYPES = (torch.float32, torch.bfloat16)


def _has_native() -> bool:
    from .. import ops
    return ops.native() is not None


class _Lazy:
    def __bool__(self):
        return _has_native()

    def __repr__(self):
        return repr(bool(self))


HAS_NATIVE = _Lazy()


def set_backend(name: str) -> None:
    global _BACKEND
    if name == "triton":
        name = "native"
    if name not in ("auto", "fallback", "native"):
        raise ValueError(f"unknown kernel backend {name!r}; use auto|fallback|native")
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


def stats() -> dict:
    return {"fast": _COUNTS["fast"], "fallback": _COUNTS["fallback"], "reasons": dict(_COUNTS["reason"])}


def reset_stats() -> None:
    _COUNTS["fast"] = 0
    _COUNTS["fallback"] = 0
    _COUNTS["reason"] = {}


def tracing() -> bool:
    try:
        return torch.compiler.is_compiling()
    except Exception:  # pragma: no cover
        return False


def use_custom_ops(flag: "bool | None" = None) -> bool:
    """Route the kernels through ``torch.library`` custom ops (for export); returns the setting."""
    global _FORCE_CUSTOM_OPS
    if flag is not None:
        _FORCE_CUSTOM_OPS = bool(flag)
    return _FORCE_CUSTOM_OPS


def _miss(why: str) -> bool:
    if not tracing():
        _COUNTS["fallback"] += 1
        _COUNTS["reason"][why] = _COUNTS["reason"].get(why, 0) + 1
    return False


def fast_ok(*tensors) -> bool:
    """Can the CUDA kernels serve these tensors right now? Records the decision in ``stats()``."""
    if _BACKEND == "fallback":
        return _miss("backend=fallback")
    if tracing():
        return False
    for t in tensors:
        if not isinstance(t, torch.Tensor):
            continue
        if not t.is_cuda:
            if _BACKEND == "native":
                raise RuntimeError("kernel backend 'native' needs CUDA tensors")
            return _miss("not cuda")
        if t.dtype not in _DTYPES:
            return _miss(f"dtype {t.dtype}")
    from .. import ops
    if not ops.available():
        if _BACKEND == "native" or torch.cuda.is_available():
            ops.require()          # a GPU box without the extension is an error, not a fallback
        return _miss("no native extension")
    _COUNTS["fast"] += 1
    return True
