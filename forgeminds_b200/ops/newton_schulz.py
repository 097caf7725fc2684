"""Quintic Newton-Schulz iteration on the tcgen05 GEMM.

One iteration ``X <- a X + (b A + c A A) X`` with ``A = X X^T`` is three GEMM launches and no
elementwise kernel: the polynomial lives in the epilogues (``D = alpha * op(A) op(B)^T + beta * C``):

    A  = X X^T                      gemm(X, X)
    Bm = c * A A^T + b * A          gemm(A, A, c=A, alpha=c, beta=b)      (A is symmetric)
    X' = Bm X + a * X               gemm(Bm, X, b_mn=True, c=X, beta=a)

The reference runs the same three products through cuBLAS and two Triton elementwise kernels
(``forgemind/kernels/ns.py:155-170``).
"""
from __future__ import annotations

import torch

from . import require, status_word
from .functional import gemm

NS_A, NS_B, NS_C = 3.4445, -4.7750, 2.0315


def newton_schulz_bf16(g: torch.Tensor, steps: int = 5):
    """``g [..., m, n]`` -> orthogonalised bf16 tensor of the same shape, or ``None`` when a
    dimension does not meet the kernel's alignment (multiples of 8)."""
    shape = g.shape
    m, n = shape[-2], shape[-1]
    if m % 8 or n % 8:
        return None
    x = g.reshape(-1, m, n)
    flip = m > n
    if flip:
        x = x.mT
    x = x.to(torch.bfloat16)
    x = (x / (x.norm(dim=(-2, -1), keepdim=True) + 1e-7)).contiguous()
    r, c = x.shape[-2], x.shape[-1]
    if x.shape[0] > 1 and r % 128 == 0:
        return _batched(x, steps, flip, shape)
    out = torch.empty_like(x)
    gram = torch.empty((r, r), dtype=torch.bfloat16, device=x.device)
    poly = torch.empty_like(gram)
    for i in range(x.shape[0]):
        cur = x[i]
        nxt = out[i]
        for _ in range(steps):
            gemm(cur, cur, out=gram)
            gemm(gram, gram, out=poly, c=gram, alpha=NS_C, beta=NS_B)
            gemm(poly, cur, b_mn=True, out=nxt, c=cur, alpha=1.0, beta=NS_A)
            cur, nxt = nxt, cur
        if cur.data_ptr() != out[i].data_ptr():
            out[i].copy_(cur)
    if flip:
        out = out.mT
    return out.reshape(shape)


_tile_groups = {}


def _batched(x: torch.Tensor, steps: int, flip: bool, shape):
    """All matrices of a stack in one launch per product (row tiles of entry g use B matrix g)."""
    C = require()
    G, r, c = x.shape
    key = (G, r, x.device)
    tg = _tile_groups.get(key)
    if tg is None:
        tg = torch.arange(G, dtype=torch.int32, device=x.device).repeat_interleave(r // 128).contiguous()
        _tile_groups[key] = tg
    st = status_word(x.device)
    cur, nxt = x, torch.empty_like(x)
    gram = torch.empty((G, r, r), dtype=torch.bfloat16, device=x.device)
    poly = torch.empty_like(gram)
    for _ in range(steps):
        C.gemm_batched(cur, cur, gram, None, False, 1.0, 0.0, tg, st)
        C.gemm_batched(gram, gram, poly, gram, False, NS_C, NS_B, tg, st)
        C.gemm_batched(poly, cur, nxt, cur, True, 1.0, NS_A, tg, st)
        cur, nxt = nxt, cur
    out = cur.mT if flip else cur
    return out.reshape(shape)
