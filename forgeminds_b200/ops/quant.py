"""Quantised matrix products on the 8-bit tensor-core paths (``csrc/gemm8_sm100.cu``).

``qmatmul(a, weight, mode, block, transpose_w)`` is what :mod:`forgeminds_b200.quant` calls on a
B200: both operands are quantised on the device and multiplied by the int8 (``kind::i8``) or fp8
(``kind::f8f6f4``) tcgen05 kernel.

* ``int8``: one scale per row of each operand (per token, per output channel); int32 accumulation in
  TMEM, scales applied in the epilogue.
* ``fp8``: e4m3 with one scale per row and ``block``-wide K group for the activations and one scale
  per ``block x block`` tile for the weights; each K block is accumulated in its own TMEM buffer and
  added, scaled, in fp32. ``block`` other than 128 falls back to row scales for both operands.

Quantised weights are cached per parameter and refreshed after every optimizer step. The reference
delegates these products to torchao / Transformer Engine (``forgemind/quant.py:93-154``).
"""
from __future__ import annotations

import torch

from . import functional as Fn
from . import require, status_word

KINDS = {"int8": 0, "fp8": 1}


def _cached_weight(weight, mode: str, block: int, transposed: bool):
    """Quantised ``weight`` (``[N, K]``, K-major) or ``weight.T``; cached until the weights change."""
    C = require()
    key = (mode, block, transposed)
    cache = getattr(weight, "_fm_qcache", None)
    stamp = (weight._version, Fn._weights_epoch)
    if cache is not None and cache.get("stamp") == stamp and key in cache:
        return cache[key]
    if cache is None or cache.get("stamp") != stamp:
        cache = {"stamp": stamp}
        try:
            weight._fm_qcache = cache
        except Exception:                        # noqa: BLE001 - not every tensor takes attributes
            pass
    shadow = getattr(weight, "_fm_shadow", None)
    if shadow is not None and len(shadow) == 2:
        # a flat store owns this parameter: its bf16 copy is complete on every rank, the fp32 master may be sharded
        w = Fn.bf16_of(weight)
    else:
        w = weight.detach()
    if transposed:
        w = w.t()
    w = w.contiguous()
    if mode == "fp8" and block == 128:
        entry = tuple(C.quant_tiles_fp8(w))
    else:
        entry = tuple(C.quant_rows(w, KINDS[mode], 0))
    cache[key] = entry
    return entry


def _cached_fused(weights, mode: str, block: int, transposed: bool):
    """Quantised ``cat(weights)`` (``[sum N_i, K]``) or its transpose, cached on the first weight until any
    optimizer steps. In a flat parameter store the bf16 copies of q|k|v and of gate|up are neighbours, so
    the concatenation is a view."""
    C = require()
    head = weights[0]
    key = ("fused", len(weights), mode, block, transposed)
    stamp = (tuple(w._version for w in weights), Fn._weights_epoch)
    cache = getattr(head, "_fm_qcache_multi", None)
    if cache is None or cache.get("stamp") != stamp:
        cache = {"stamp": stamp}
        head._fm_qcache_multi = cache
    if key not in cache:
        w = Fn.fused_bf16(weights)
        w = (w.t() if transposed else w).contiguous()
        cache[key] = tuple(C.quant_tiles_fp8(w)) if (mode == "fp8" and block == 128) else tuple(C.quant_rows(w, KINDS[mode], 0))
    return cache[key]


class _QLinearMulti(torch.autograd.Function):
    """``x @ cat(weights).T`` on the 8-bit tensor-core path as ONE product: the activations are quantised
    once for all the projections that share them, the input gradient is one product against the
    concatenated weights, the weight gradient one bf16 product that accumulates into the (adjacent) fp32
    gradient buffers. Used for q|k|v and gate|up of the quantised blocks."""

    @staticmethod
    def forward(ctx, x, mode, block, *weights):
        C = require()
        x2 = Fn._rows(x)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        blocked = mode == "fp8" and block == 128
        wq, ws = _cached_fused(weights, mode, block, transposed=False)
        aq, a_s = C.quant_rows(x2, KINDS[mode], 128 if blocked else 0)
        y = C.gemm8(aq, wq, a_s, ws, KINDS[mode], False, status_word(x.device))
        ctx.save_for_backward(x2)
        ctx.weights, ctx.mode, ctx.block, ctx.x_shape = weights, mode, block, x.shape
        # reshape the fresh tensor itself: a view returned from a Function could not be updated in place (RoPE does)
        return y.resize_(*x.shape[:-1], y.shape[-1])

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy):
        C = require()
        (x2,) = ctx.saved_tensors
        weights, mode, block = ctx.weights, ctx.mode, ctx.block
        dy2 = Fn._rows(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            blocked = mode == "fp8" and block == 128
            wq_t, ws_t = _cached_fused(weights, mode, block, transposed=True)
            gq, g_s = C.quant_rows(dy2, KINDS[mode], 128 if blocked else 0)
            dx = C.gemm8(gq, wq_t, g_s, ws_t, KINDS[mode], False, status_word(dy.device)).view(ctx.x_shape)
        grads = Fn._weight_grads(ctx.needs_input_grad[3:], weights, dy2, x2)
        return (dx, None, None, *grads)


def qlinear_multi(x, weights, mode: str, block: int = 128):
    """Fused quantised projection: ``x @ cat(weights).T`` (bf16 result), weights in ``nn.Linear`` layout."""
    k = x.shape[-1]
    if k % 16 or any(w.shape[0] % 8 for w in weights):
        raise ValueError("quantised products need an inner dimension that is a multiple of 16 and output widths "
                         "that are multiples of 8")
    return _QLinearMulti.apply(x, mode, int(block), *weights)


def qmatmul(a: torch.Tensor, weight: torch.Tensor, mode: str, block: int, transpose_w: bool) -> torch.Tensor:
    """``a @ weight.T`` (``transpose_w``) or ``a @ weight`` with both operands quantised; bf16 result."""
    C = require()
    if mode not in KINDS:
        raise ValueError(f"unknown quantisation mode {mode!r}")
    a2 = a.detach()
    if a2.dtype not in (torch.bfloat16, torch.float32):
        a2 = a2.to(torch.bfloat16)
    if a2.stride(-1) != 1:
        a2 = a2.contiguous()
    k = a2.shape[1]
    if k % 16:
        raise ValueError("quantised products need an inner dimension that is a multiple of 16")
    blocked = mode == "fp8" and block == 128
    wq, ws = _cached_weight(weight, mode, block, transposed=not transpose_w)
    aq, a_s = C.quant_rows(a2, KINDS[mode], 128 if blocked else 0)
    n = wq.shape[0]
    if n % 8:
        raise ValueError("quantised products need an output width that is a multiple of 8")
    return C.gemm8(aq, wq, a_s, ws, KINDS[mode], False, status_word(a.device))
