"""Building blocks for user architectures that run on the fused kernels: :class:`RMSNorm`, :class:`SwiGLU`.

Drop-in ``nn.Module``s: on a B200 their forward goes through :mod:`forgeminds_b200.kernels` (hand-written
sm_100a kernels, fp32 accumulation, one rounding at the store), anywhere else through the PyTorch
statement of the same arithmetic. State-dict contract (the reference's ``forgemind/nn.py:82-217``):
``RMSNorm`` has the single parameter ``weight [dim]`` of ``torch.nn.RMSNorm`` and loads from / into one;
``SwiGLU`` has ``w1, w3, w2`` (``nn.Linear`` layout) or, when ``split=True``, ``gate_up, w2`` with
``gate_up.weight = cat(w1.weight, w3.weight)``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import kernels as K

__all__ = ["RMSNorm", "SwiGLU"]


def _positive(name: str, value) -> int:
    n = int(value)
    if n < 1:
        raise ValueError(f"{name} must be a positive integer, got {value!r}")
    return n


class RMSNorm(nn.Module):
    """Root-mean-square normalisation of the last dimension, ``y = x / sqrt(mean(x^2) + eps) * weight``.

    ``forward_with_residual(x, r)`` fuses the residual add that usually precedes a pre-norm block: it
    returns ``(norm(x + r), x + r)`` from a single pass over the row.
    """

    def __init__(self, dim: int, eps: float = 1e-6, elementwise_affine: bool = True, device=None, dtype=None):
        super().__init__()
        self.dim = _positive("RMSNorm dim", dim)
        self.eps = float(eps)
        self.elementwise_affine = bool(elementwise_affine)
        gain = nn.Parameter(torch.ones(self.dim, device=device, dtype=dtype)) if self.elementwise_affine else None
        self.register_parameter("weight", gain)

    def extra_repr(self) -> str:
        affine = "" if self.elementwise_affine else ", no weight"
        return f"dim={self.dim}, eps={self.eps:g}{affine}"

    def _gain_for(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.dim:
            raise ValueError(f"input of shape {tuple(x.shape)} cannot be normalised by RMSNorm(dim={self.dim}): "
                             "the last dimension must equal dim")
        if self.weight is None:
            return x.new_ones(self.dim)
        return self.weight.to(x.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return K.rms_norm(x, self._gain_for(x), self.eps)

    def forward_with_residual(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        gain = self._gain_for(x)
        if residual is None:
            return K.rms_norm(x, gain, self.eps), x
        if tuple(residual.shape) != tuple(x.shape):
            raise ValueError(f"residual {tuple(residual.shape)} and input {tuple(x.shape)} must have the same shape")
        total, normed = K.add_rms_norm(x, residual, gain, self.eps)
        return normed, total


class SwiGLU(nn.Module):
    """Gated MLP ``w2(silu(w1 x) * (w3 x))``.

    ``split=True`` keeps gate and up as the two halves of one ``gate_up`` projection, so the block is
    two GEMMs instead of three and the activation reads one buffer. :meth:`to_split` converts an
    existing module (in place, or as a copy) without changing what it computes.
    """

    def __init__(self, dim: int, hidden: Optional[int] = None, bias: bool = False, split: bool = False,
                 device=None, dtype=None):
        super().__init__()
        self.dim = _positive("SwiGLU dim", dim)
        self.hidden = _positive("SwiGLU hidden", 4 * self.dim if hidden is None else hidden)
        self.split = bool(split)
        make = lambda fan_in, fan_out: nn.Linear(fan_in, fan_out, bias=bias, device=device, dtype=dtype)  # noqa: E731
        if self.split:
            self.gate_up = make(self.dim, 2 * self.hidden)
        else:
            self.w1, self.w3 = make(self.dim, self.hidden), make(self.dim, self.hidden)
        self.w2 = make(self.hidden, self.dim)

    def extra_repr(self) -> str:
        return f"dim={self.dim}, hidden={self.hidden}, layout={'gate_up|w2' if self.split else 'w1,w3|w2'}"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.split:
            act = K.swiglu_split(self.gate_up(x))
        else:
            act = K.swiglu(self.w1(x), self.w3(x))
        return self.w2(act)

    @torch.no_grad()
    def to_split(self, inplace: bool = True) -> "SwiGLU":
        if self.split:
            return self
        gate, up = self.w1, self.w3
        with_bias = gate.bias is not None
        if with_bias != (up.bias is not None):
            raise ValueError("cannot merge w1 and w3: one has a bias and the other does not")
        ref = gate.weight
        merged = SwiGLU(self.dim, self.hidden, bias=with_bias, split=True, device=ref.device, dtype=ref.dtype)
        merged.gate_up.weight[:self.hidden] = gate.weight
        merged.gate_up.weight[self.hidden:] = up.weight
        if with_bias:
            merged.gate_up.bias[:self.hidden] = gate.bias
            merged.gate_up.bias[self.hidden:] = up.bias
        if not inplace:
            has_out_bias = self.w2.bias is not None
            if has_out_bias != with_bias:
                merged.w2 = nn.Linear(self.hidden, self.dim, bias=has_out_bias, device=ref.device, dtype=ref.dtype)
            merged.w2.load_state_dict(self.w2.state_dict())
            merged.train(self.training)
            return merged
        self.gate_up = merged.gate_up
        del self.w1, self.w3
        self.split = True
        return self
