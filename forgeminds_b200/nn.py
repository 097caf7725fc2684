"""Composable blocks backed by the fused kernels: :class:`RMSNorm` and :class:`SwiGLU`.

Both are ordinary ``nn.Module``s usable in any architecture; on a B200 they call the CUDA kernels,
elsewhere the equivalent PyTorch expressions. ``RMSNorm`` keeps ``torch.nn.RMSNorm``'s parameter
name and shape; ``SwiGLU(split=True)`` holds one ``gate_up`` projection instead of ``w1``/``w3``.
Interface as in the reference's ``forgemind/nn.py:82-217``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .kernels import add_rms_norm, rms_norm, swiglu, swiglu_split

__all__ = ["RMSNorm", "SwiGLU"]


class RMSNorm(nn.Module):
    """``x * rsqrt(mean(x^2) + eps) * weight`` over the last dimension."""

    def __init__(self, dim: int, eps: float = 1e-6, elementwise_affine: bool = True, device=None, dtype=None):
        super().__init__()
        self.dim = int(dim)
        if self.dim <= 0:
            raise ValueError(f"RMSNorm needs dim > 0, got {dim}")
        self.eps = float(eps)
        self.elementwise_affine = bool(elementwise_affine)
        if self.elementwise_affine:
            self.weight = nn.Parameter(torch.ones(self.dim, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)

    def extra_repr(self) -> str:
        return f"{self.dim}, eps={self.eps}, elementwise_affine={self.elementwise_affine}"

    def _scale(self, x):
        if self.weight is None:
            return torch.ones(self.dim, device=x.device, dtype=x.dtype)
        return self.weight if self.weight.dtype == x.dtype else self.weight.to(x.dtype)

    def _check(self, x) -> None:
        if x.shape[-1] != self.dim:
            raise ValueError(f"RMSNorm({self.dim}) got last dim {x.shape[-1]}; the norm runs over the last "
                             f"dimension of [..., {self.dim}]")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self._check(x)
        return rms_norm(x, self._scale(x), self.eps)

    def forward_with_residual(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        """``(normed, x + residual)`` with the sum written once and normalised in the same pass."""
        self._check(x)
        if residual is None:
            residual = torch.zeros_like(x)
        elif residual.shape != x.shape:
            raise ValueError(f"residual shape {tuple(residual.shape)} does not match x {tuple(x.shape)}")
        summed, normed = add_rms_norm(x, residual, self._scale(x), self.eps)
        return normed, summed


class SwiGLU(nn.Module):
    """``w2(silu(w1 x) * w3 x)``; with ``split=True`` the gate and up projections are one GEMM."""

    def __init__(self, dim: int, hidden: int | None = None, bias: bool = False, split: bool = False,
                 device=None, dtype=None):
        super().__init__()
        self.dim = int(dim)
        self.hidden = int(hidden if hidden is not None else 4 * dim)
        if self.dim <= 0 or self.hidden <= 0:
            raise ValueError(f"SwiGLU needs dim > 0 and hidden > 0, got dim={dim}, hidden={hidden}")
        self.split = bool(split)
        kw = dict(bias=bias, device=device, dtype=dtype)
        if self.split:
            self.gate_up = nn.Linear(self.dim, 2 * self.hidden, **kw)
        else:
            self.w1 = nn.Linear(self.dim, self.hidden, **kw)
            self.w3 = nn.Linear(self.dim, self.hidden, **kw)
        self.w2 = nn.Linear(self.hidden, self.dim, **kw)

    def extra_repr(self) -> str:
        return f"{self.dim} -> {self.hidden} -> {self.dim}, split={self.split}"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.split:
            return self.w2(swiglu_split(self.gate_up(x)))
        return self.w2(swiglu(self.w1(x), self.w3(x)))

    @torch.no_grad()
    def to_split(self, inplace: bool = True) -> "SwiGLU":
        """Concatenate ``w1|w3`` into ``gate_up`` (same function, renamed parameters)."""
        if self.split:
            return self
        if (self.w1.bias is None) != (self.w3.bias is None):
            raise ValueError("to_split() needs both projections to have a bias, or neither")
        target = self
        if not inplace:
            target = SwiGLU(self.dim, self.hidden, bias=self.w2.bias is not None, split=False,
                            device=self.w2.weight.device, dtype=self.w2.weight.dtype)
            target.w2.load_state_dict(self.w2.state_dict())
        fused = nn.Linear(self.dim, 2 * self.hidden, bias=self.w1.bias is not None,
                          device=self.w1.weight.device, dtype=self.w1.weight.dtype)
        fused.weight.copy_(torch.cat([self.w1.weight, self.w3.weight], dim=0))
        if fused.bias is not None:
            fused.bias.copy_(torch.cat([self.w1.bias, self.w3.bias], dim=0))
        del target.w1, target.w3
        target.gate_up = fused
        target.split = True
        return target
