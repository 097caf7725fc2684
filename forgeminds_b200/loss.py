"""Cross-entropy over large vocabularies without a full ``[tokens, vocab]`` logits tensor.

``chunked_cross_entropy`` is the PyTorch path (CPU, fp32): logits exist one chunk of rows at a
time and are recomputed in the backward (non-reentrant checkpoint). On a B200 with bf16
activations the model calls :func:`forgeminds_b200.ops.functional.linear_cross_entropy` instead,
which writes the gradient of each logits chunk in place and runs the two gradient GEMMs once.
Semantics (mean over labels != ignore_index, fp32 result) follow the reference's
``forgemind/loss.py:23-70``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

__all__ = ["chunked_cross_entropy", "logits_cross_entropy", "fused_linear_cross_entropy"]


def _count_valid(labels, ignore_index):
    return (labels != ignore_index).sum().clamp(min=1).to(torch.float32)


def chunked_cross_entropy(h, weight, labels, chunk: int = 4096, ignore_index: int = -100):
    """Mean CE of ``h @ weight.T`` against ``labels``; returns a 0-dim fp32 tensor."""
    rows = h.reshape(-1, h.shape[-1])
    y = labels.reshape(-1)
    denom = _count_valid(y, ignore_index)
    w = weight if weight.dtype == rows.dtype else weight.to(rows.dtype)
    track = torch.is_grad_enabled() and (rows.requires_grad or weight.requires_grad)

    def chunk_sum(hc, yc):
        return F.cross_entropy(F.linear(hc, w), yc, ignore_index=ignore_index, reduction="sum").float()

    acc = None
    for lo in range(0, rows.shape[0], chunk):
        hc, yc = rows[lo:lo + chunk], y[lo:lo + chunk]
        piece = checkpoint(chunk_sum, hc, yc, use_reentrant=False) if track else chunk_sum(hc, yc)
        acc = piece if acc is None else acc + piece
    if acc is None:     # no tokens at all
        acc = rows.new_zeros((), dtype=torch.float32)
        return acc.requires_grad_(True) if track else acc
    return acc / denom


def logits_cross_entropy(logits, labels, ignore_index: int = -100, chunk: int = 4096):
    """Mean CE when the logits already exist (last pipeline stage); reduced in row chunks so that
    no second full-size fp32 buffer appears."""
    flat = logits.reshape(-1, logits.shape[-1])
    y = labels.reshape(-1)
    denom = _count_valid(y, ignore_index)
    acc = None
    for lo in range(0, flat.shape[0], chunk):
        piece = F.cross_entropy(flat[lo:lo + chunk], y[lo:lo + chunk], ignore_index=ignore_index,
                                reduction="sum").float()
        acc = piece if acc is None else acc + piece
    if acc is None:
        return flat.new_zeros((), dtype=torch.float32)
    return acc / denom


def fused_linear_cross_entropy(h, weight, labels, chunk: int = 4096, ignore_index: int = -100):
    """Dispatch: sm_100a kernels for bf16 CUDA activations, the chunked PyTorch path otherwise."""
    if h.is_cuda and h.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0 and h.shape[-1] % 8 == 0:
        from . import ops
        if ops.available():
            from .ops.functional import linear_cross_entropy
            return linear_cross_entropy(h, weight, labels, chunk, ignore_index)
    return chunked_cross_entropy(h, weight, labels, chunk, ignore_index)
