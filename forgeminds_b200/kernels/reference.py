"""Plain-PyTorch statements of every kernel in this package.

They fix the semantics the CUDA kernels must match -- accumulate in fp32 (fp64 inputs stay fp64),
round once when storing, output dtype equals input dtype -- and are the CPU path of the public
functions. Counterpart of the reference's ``forgemind/kernels/_fallback.py:15-109``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def _wide(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype in (torch.float32, torch.float64) else t.float()


def rms_norm(x, w, eps: float = 1e-6):
    xf = _wide(x)
    inv = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
    return (xf * inv * _wide(w)).to(x.dtype)


def add_rms_norm(x, delta, w, eps: float = 1e-6):
    summed = x + delta
    return summed, rms_norm(summed, w, eps)


def rotate_half_split(y, cos, sin):
    a, b = y.chunk(2, dim=-1)
    return torch.cat((a * cos - b * sin, a * sin + b * cos), dim=-1)


def qk_norm_rope(x, w, cos, sin, eps: float = 1e-6):
    """Per-head RMSNorm over the head dim of ``x [B,T,H,D]`` followed by half-split rotation."""
    xf = _wide(x)
    inv = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
    return rotate_half_split(xf * inv * _wide(w), cos, sin).to(x.dtype)


def swiglu(gate, up):
    return (F.silu(_wide(gate)) * _wide(up)).to(gate.dtype)


def swiglu_split(x):
    h = x.shape[-1] // 2
    return swiglu(x[..., :h], x[..., h:])


def kl_div_logits(student, teacher, reduction: str = "mean"):
    """``KL(softmax(teacher) || softmax(student))`` over the last dim and its gradient with respect
    to the student logits (already scaled for the chosen reduction)."""
    log_s = torch.log_softmax(_wide(student), dim=-1)
    log_t = torch.log_softmax(_wide(teacher), dim=-1)
    p_t = log_t.exp()
    rows = (p_t * (log_t - log_s)).sum(dim=-1)
    if reduction == "none":
        loss, scale = rows, 1.0
    elif reduction == "sum":
        loss, scale = rows.sum(), 1.0
    else:
        scale = 1.0 / max(1, rows.numel())
        loss = rows.sum() * scale
    return loss, ((log_s.exp() - p_t) * scale).to(student.dtype)


def kl_distill_loss(hs, ht, w, teacher_head, chunk: int = 4096):
    """Mean KL of ``softmax(teacher_head(ht)) || softmax(hs @ w.T)``; gradients reach ``hs`` and ``w``
    only. Student logits exist one chunk of rows at a time."""
    s2 = hs.reshape(-1, hs.shape[-1])
    t2 = ht.reshape(-1, ht.shape[-1])
    rows = s2.shape[0]
    total = None
    for lo in range(0, rows, chunk):
        hi = min(rows, lo + chunk)
        with torch.no_grad():
            t_logits = teacher_head(t2[lo:hi]).detach()
        part = kl_div_logits(s2[lo:hi] @ w.t(), t_logits, "sum")[0]
        total = part if total is None else total + part
    return total / rows


def newton_schulz(g, steps: int = 5, dtype=None):
    """Quintic Newton-Schulz orthogonalisation of ``g [..., m, n]`` (Gram matrix on the short side,
    Frobenius pre-scaling; coefficients 3.4445, -4.7750, 2.0315)."""
    a, b, c = NS_COEFFS
    shape = g.shape
    work = torch.float32 if g.dtype == torch.float32 else torch.bfloat16
    if dtype is not None:
        work = dtype
    x = g.reshape(-1, shape[-2], shape[-1])
    flip = shape[-2] > shape[-1]
    if flip:
        x = x.mT
    x = x.to(work)
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        gram = x @ x.mT
        x = a * x + (b * gram + c * (gram @ gram)) @ x
    if flip:
        x = x.mT
    return x.reshape(shape)


def topk(x, k: int):
    """Top-k of the last dim: values descending, NaN largest, equal values by ascending index."""
    xf = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
    key = torch.where(torch.isnan(xf), torch.full_like(xf, float("inf")), xf)
    order = torch.sort(key, dim=-1, descending=True, stable=True).indices[..., :k]
    return torch.gather(x, -1, order), order


def softmax(x):
    return torch.softmax(x, dim=-1)
