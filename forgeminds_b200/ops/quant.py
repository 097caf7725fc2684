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
