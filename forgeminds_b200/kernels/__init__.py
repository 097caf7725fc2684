"""Fused kernels with a functional interface.

Each function replaces an eager PyTorch expression, keeps its autograd contract and picks one of
two implementations per call:

* the hand-written sm_100a kernel (CUDA tensors of a supported dtype on a compute-capability-10
  device, backend not forced to ``"fallback"``), or
* the PyTorch statement in :mod:`forgeminds_b200.kernels.reference` (CPU, other dtypes, while
  ``torch.compile`` traces).

``stats()`` reports how often each path ran and why. Public names follow the reference's
``forgemind/kernels/__init__.py:42-48``.

    import forgeminds_b200 as fm
    y = fm.kernels.rms_norm(x, w, 1e-6)
    xn, y = fm.kernels.add_rms_norm(x, delta, w)
    y = fm.kernels.swiglu(gate, up);  y = fm.kernels.swiglu_split(gate_up)
    y = fm.kernels.qk_norm_rope(q, w, cos, sin)
    loss = fm.kernels.kl_distill_loss(hs, ht, w, teacher_head)
    fm.kernels.enable(model); fm.kernels.patch(model.norm); fm.kernels.revert(model)
"""
from __future__ import annotations

import torch

from . import reference as _ref
from ._state import (HAS_NATIVE, HAS_TRITON, fast_ok, get_backend, reset_stats, set_backend, stats, tracing,
                     use_custom_ops)

__all__ = [
    "HAS_TRITON", "HAS_NATIVE", "set_backend", "get_backend", "stats", "reset_stats",
    "rms_norm", "add_rms_norm", "qk_norm_rope", "swiglu", "swiglu_split",
    "kl_div_logits", "kl_div", "kl_distill_loss", "distill_kl",
    "newton_schulz", "topk", "softmax",
    "enable", "patch", "revert", "available", "use_custom_ops",
]

MAX_K = 512


def available() -> bool:
    """True when the CUDA kernels can run on this machine."""
    from .. import ops
    return ops.available()


def _fn():
    from ..ops import functional
    return functional


# ------------------------------------------------------------------------------ norms
def _use_ops() -> bool:
    """Whether the public functions go through the ``torch.library`` forms (``kernels/_ops.py``)."""
    from . import _ops
    return use_custom_ops() or _ops.env_default()


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w`` over the last dimension."""
    if _use_ops():
        from . import _ops
        return _ops.rms_norm_op(x, w, float(eps))
    return _rms_norm_eager(x, w, eps)


def _rms_norm_eager(x, w, eps=1e-6):
    if x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384 and fast_ok(x, w):
        return _fn().rms_norm(x, w, eps)
    return _ref.rms_norm(x, w, eps)


def add_rms_norm(x: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float = 1e-6):
    """Residual add and norm in one pass: returns ``(x + delta, rms_norm(x + delta, w))``."""
    if _use_ops() and x.shape == delta.shape:
        from . import _ops
        return _ops.add_rms_norm_op(x, delta, w, float(eps))
    return _add_rms_norm_eager(x, delta, w, eps)


def _add_rms_norm_eager(x, delta, w, eps=1e-6):
    if x.shape == delta.shape and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384 and fast_ok(x, delta, w):
        return _fn().add_rms_norm(x, delta, w, eps)
    return _ref.add_rms_norm(x, delta, w, eps)


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, cos, sin, eps):
        from .. import ops
        y, rstd = ops.require().qk_norm_rope_fwd(x.contiguous(), w.detach().contiguous(), cos, sin, eps)
        ctx.save_for_backward(x, w.detach(), cos, sin, rstd)
        ctx.w_dtype = w.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        from .. import ops
        x, w, cos, sin, rstd = ctx.saved_tensors
        dx, dw = ops.require().qk_norm_rope_bwd(dy.contiguous(), x.contiguous(), w.contiguous(), cos, sin, rstd)
        return dx, dw.to(ctx.w_dtype), None, None, None


def _rope_table(t: torch.Tensor, T: int, half: int):
    """Accepts [T, hd/2] or the broadcastable [1, T, 1, hd/2]; returns contiguous fp32 [T, hd/2]."""
    if t.numel() != T * half:
        return None
    return t.reshape(T, half).to(torch.float32).contiguous()


def qk_norm_rope(x: torch.Tensor, w: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 eps: float = 1e-6) -> torch.Tensor:
    """Per-head RMSNorm over the head dimension of ``x [B,T,H,D]``, then half-split RoPE."""
    if x.dim() == 4 and x.shape[-1] % 16 == 0 and x.shape[-1] <= 128 and fast_ok(x, w):
        T, half = x.shape[1], x.shape[-1] // 2
        c, s = _rope_table(cos, T, half), _rope_table(sin, T, half)
        if c is not None and s is not None and w.dtype in (x.dtype, torch.float32):
            return _QKNormRope.apply(x, w, c, s, eps)
    return _ref.qk_norm_rope(x, w, cos, sin, eps)


# ------------------------------------------------------------------------------ SwiGLU
def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for two tensors of the same shape (no broadcasting: a mismatch is almost
    always a wiring mistake and would silently multiply the cost)."""
    if gate.shape != up.shape:
        raise ValueError(f"swiglu needs gate and up of one shape, got {tuple(gate.shape)} and {tuple(up.shape)}")
    if _use_ops() and gate.shape == up.shape and gate.dtype == up.dtype:
        from . import _ops
        return _ops.swiglu_op(gate, up)
    return _swiglu_eager(gate, up)


def _swiglu_eager(gate, up):
    if gate.shape == up.shape and gate.shape[-1] % 8 == 0 and gate.dtype == up.dtype and fast_ok(gate, up):
        return _fn().swiglu(gate, up)
    return _ref.swiglu(gate, up)


def swiglu_split(x: torch.Tensor) -> torch.Tensor:
    """``silu(x[..., :h]) * x[..., h:]`` for the output of a fused gate|up projection."""
    if x.shape[-1] % 2:
        raise ValueError(f"swiglu_split halves the last dimension into gate and up; it is odd here: {tuple(x.shape)}")
    if x.shape[-1] % 16 == 0 and fast_ok(x):
        return _fn().swiglu_split(x)
    return _ref.swiglu_split(x)


# ------------------------------------------------------------------------------ KL
class _KLDiv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, student, teacher, reduction, reuse):
        from .. import ops
        V = student.shape[-1]
        rows = student.numel() // V
        scale = 1.0 / rows if reduction == "mean" else 1.0
        need = student.requires_grad
        row_loss, grad = ops.require().kl_fwd_bwd(student.contiguous(), teacher.contiguous(), scale, need,
                                                  bool(reuse and need))
        ctx.save_for_backward(grad if need else None)
        ctx.shape = student.shape
        ctx.reduction = reduction
        if reduction == "none":
            return row_loss.view(student.shape[:-1])
        total = row_loss.sum()
        return total * scale if reduction == "mean" else total

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        if grad is None:
            return None, None, None, None
        if ctx.reduction == "none":
            grad = grad.view(ctx.shape) * g.unsqueeze(-1).to(grad.dtype)
        else:
            grad = grad.view(ctx.shape) * g.to(grad.dtype)
        return grad, None, None, None


def kl_div_logits(student: torch.Tensor, teacher: torch.Tensor, reduction: str = "mean",
                  grad_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``KL(softmax(teacher) || softmax(student))`` over the last dim; the teacher is a constant."""
    if reduction not in ("mean", "sum", "none"):
        raise ValueError(f"reduction must be mean|sum|none, got {reduction!r}")
    if (student.shape == teacher.shape and student.shape[-1] > 0 and student.dtype == teacher.dtype
            and fast_ok(student, teacher)):
        return _KLDiv.apply(student, teacher.detach(), reduction, False)
    return _ref.kl_div_logits(student, teacher.detach(), reduction)[0]


def kl_distill_loss(hs: torch.Tensor, ht: torch.Tensor, w: torch.Tensor, teacher_head,
                    chunk: int = 4096) -> torch.Tensor:
    """Mean KL of ``softmax(teacher_head(ht)) || softmax(hs @ w.T)``; the teacher runs without grad."""
    if not fast_ok(hs, ht):
        return _ref.kl_distill_loss(hs, ht, w, teacher_head, chunk)
    s2 = hs.reshape(-1, hs.shape[-1])
    t2 = ht.reshape(-1, ht.shape[-1])
    rows = s2.shape[0]
    total = None
    for lo in range(0, rows, chunk):
        hi = min(rows, lo + chunk)
        with torch.no_grad():
            t_logits = teacher_head(t2[lo:hi]).detach()
        s_logits = s2[lo:hi] @ w.t()
        if s_logits.dtype != t_logits.dtype:
            t_logits = t_logits.to(s_logits.dtype)
        part = _KLDiv.apply(s_logits, t_logits, "sum", True)
        total = part if total is None else total + part
    return total / rows


kl_div = kl_div_logits
distill_kl = kl_distill_loss


# ------------------------------------------------------------------------------ Newton-Schulz
def newton_schulz(g: torch.Tensor, steps: int = 5, dtype: torch.dtype | None = None,
                  fused: bool = True) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation of ``g [..., m, n]`` (not differentiable).

    The result has the compute dtype: fp32 for fp32 inputs, bf16 otherwise, or ``dtype``.
    On the GPU the three products of an iteration run on the tcgen05 GEMM with the polynomial
    folded into their epilogues (``alpha * A B^T + beta * C``)."""
    if g.ndim < 2:
        raise ValueError(f"newton_schulz needs ndim >= 2 (a matrix), got shape {tuple(g.shape)}")
    if steps < 1:
        raise ValueError(f"steps must be >= 1, got {steps}")
    if dtype is not None and dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"dtype must be float32/float16/bfloat16, got {dtype}")
    with torch.no_grad():
        work = dtype if dtype is not None else (torch.float32 if g.dtype == torch.float32 else torch.bfloat16)
        if fused and work == torch.bfloat16 and g.numel() > 0 and not tracing() and fast_ok(g):
            from ..ops.newton_schulz import newton_schulz_bf16
            out = newton_schulz_bf16(g, steps)
            if out is not None:
                return out
        return _ref.newton_schulz(g, steps, dtype)


# ------------------------------------------------------------------------------ top-k / softmax
def topk(x: torch.Tensor, k: int, dim: int = -1, sorted: bool = True):
    """``torch.topk`` over the last dim with a fixed tie rule: values descending, NaN largest, equal
    values in ascending index order."""
    if x.dim() < 1:
        raise ValueError(f"topk needs ndim >= 1, got shape {tuple(x.shape)}")
    if dim not in (-1, x.dim() - 1):
        return torch.topk(x, k, dim=dim, sorted=True)
    n = x.shape[-1]
    if k < 1 or k > n:
        raise RuntimeError(f"selected index k out of range (got {k} vs {n})")
    if tracing():
        return torch.topk(x, k, dim=-1, sorted=True)
    if k <= MAX_K and x.numel() < 2 ** 31 and fast_ok(x):
        return _fn().topk_lastdim(x, k)
    if x.is_floating_point() and not x.requires_grad:
        return _ref.topk(x, k)
    return torch.topk(x, k, dim=-1, sorted=True)


def softmax(x: torch.Tensor, dim: int = -1, dtype: torch.dtype | None = None) -> torch.Tensor:
    """``torch.softmax`` over the last dim (other dims use torch)."""
    if x.dim() < 1:
        raise ValueError(f"softmax needs ndim >= 1, got shape {tuple(x.shape)}")
    if dim not in (-1, x.dim() - 1):
        return torch.softmax(x, dim=dim, dtype=dtype)
    if dtype is not None and dtype != x.dtype:
        x = x.to(dtype)
    if not tracing() and x.numel() < 2 ** 31 and fast_ok(x):
        return _fn().softmax_lastdim(x)
    return torch.softmax(x, dim=-1)


from .apply import enable, patch, revert  # noqa: E402  (needs the functions above)
