"""``torch.library`` forms of the element-wise kernels, for tracing and export.

Eager code calls the kernels through ``autograd.Function``s (cheapest call path). A traced program
(``torch.compile(fullgraph=True)``, ``torch.export``) cannot look inside those, so each op also exists as
an opaque custom op ``forgeminds_b200::<name>`` with a fake (shape / dtype) implementation and a
registered backward that is itself a custom op; ``fm.kernels.use_custom_ops(True)`` (or
``FORGEMINDS_KERNEL_OPS=1`` in the environment) routes ``fm.kernels.rms_norm`` / ``add_rms_norm`` /
``swiglu`` through them. The implementations call the same dispatch as the eager path: the CUDA
kernels where they can serve the tensors, the PyTorch statement of the op otherwise. Counterpart of
the reference's ``forgemind/kernels/_ops.py:59-145``.
"""
from __future__ import annotations

import os

import torch

from . import reference as _ref

NS = "forgeminds_b200"


def env_default() -> bool:
    return os.environ.get("FORGEMINDS_KERNEL_OPS", "0") == "1"


class _Eager:
    """The eager dispatch of the package (CUDA kernel when it can serve the tensors, PyTorch otherwise)."""

    def __getattr__(self, name):
        from .. import kernels
        return getattr(kernels, f"_{name}_eager")


def _eager():
    return _Eager()


def _rms_bwd(gy, x, w, eps):
    """Closed-form gradients of ``x * rsqrt(mean(x^2) + eps) * w`` (fp32 arithmetic, one rounding at the end).
    An op implementation runs below the autograd dispatch key, so it cannot differentiate the forward."""
    xf, gf, wf = x.float(), gy.float(), w.float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    gw_rows = gf * xf * r
    gyw = gf * wf
    gx = r * gyw - xf * r.pow(3) * (gyw * xf).mean(-1, keepdim=True)
    return gx, gw_rows.reshape(-1, x.shape[-1]).sum(0)


# ------------------------------------------------------------------------------ rms_norm
@torch.library.custom_op(f"{NS}::rms_norm", mutates_args=())
def rms_norm_op(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return _eager().rms_norm(x, w, eps)


@rms_norm_op.register_fake
def _(x, w, eps):
    return torch.empty_like(x)


@torch.library.custom_op(f"{NS}::rms_norm_bwd", mutates_args=())
def rms_norm_bwd_op(gy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    gx, gw = _rms_bwd(gy, x, w, eps)
    return gx.to(x.dtype), gw.to(w.dtype)


@rms_norm_bwd_op.register_fake
def _(gy, x, w, eps):
    return torch.empty_like(x), torch.empty_like(w)


def _rms_setup(ctx, inputs, output):
    x, w, eps = inputs
    ctx.save_for_backward(x, w)
    ctx.eps = eps


def _rms_backward(ctx, gy):
    x, w = ctx.saved_tensors
    gx, gw = rms_norm_bwd_op(gy.contiguous(), x, w, ctx.eps)
    return gx, gw, None


rms_norm_op.register_autograd(_rms_backward, setup_context=_rms_setup)


# ------------------------------------------------------------------------------ add_rms_norm
@torch.library.custom_op(f"{NS}::add_rms_norm", mutates_args=())
def add_rms_norm_op(x: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    s, y = _eager().add_rms_norm(x, delta, w, eps)
    return s, y


@add_rms_norm_op.register_fake
def _(x, delta, w, eps):
    return torch.empty_like(x), torch.empty_like(x)


@torch.library.custom_op(f"{NS}::add_rms_norm_bwd", mutates_args=())
def add_rms_norm_bwd_op(gs: torch.Tensor, gy: torch.Tensor, x: torch.Tensor, delta: torch.Tensor, w: torch.Tensor,
                        eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    gx, gw = _rms_bwd(gy, (x.float() + delta.float()).to(x.dtype), w, eps)
    return (gx + gs.float()).to(x.dtype), gw.to(w.dtype)       # d/dx == d/ddelta: both enter through the sum


@add_rms_norm_bwd_op.register_fake
def _(gs, gy, x, delta, w, eps):
    return torch.empty_like(x), torch.empty_like(w)


def _arn_setup(ctx, inputs, output):
    x, delta, w, eps = inputs
    ctx.save_for_backward(x, delta, w)
    ctx.eps = eps


def _arn_backward(ctx, gs, gy):
    x, delta, w = ctx.saved_tensors
    gs = torch.zeros_like(x) if gs is None else gs.contiguous()
    gy = torch.zeros_like(x) if gy is None else gy.contiguous()
    gx, gw = add_rms_norm_bwd_op(gs, gy, x, delta, w, ctx.eps)
    return gx, gx, gw, None


add_rms_norm_op.register_autograd(_arn_backward, setup_context=_arn_setup)


# ------------------------------------------------------------------------------ swiglu
@torch.library.custom_op(f"{NS}::swiglu", mutates_args=())
def swiglu_op(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return _eager().swiglu(gate, up)


@swiglu_op.register_fake
def _(gate, up):
    return torch.empty_like(gate)


@torch.library.custom_op(f"{NS}::swiglu_bwd", mutates_args=())
def swiglu_bwd_op(gy: torch.Tensor, gate: torch.Tensor, up: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    g, u, v = gate.float(), up.float(), gy.float()
    sig = torch.sigmoid(g)
    return (v * u * sig * (1 + g * (1 - sig))).to(gate.dtype), (v * g * sig).to(up.dtype)


@swiglu_bwd_op.register_fake
def _(gy, gate, up):
    return torch.empty_like(gate), torch.empty_like(up)


def _sw_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _sw_backward(ctx, gy):
    gate, up = ctx.saved_tensors
    return swiglu_bwd_op(gy.contiguous(), gate, up)


swiglu_op.register_autograd(_sw_backward, setup_context=_sw_setup)
