"""Quantised training: block-scaled FP8 and INT8 linear layers.

``quantize_model(model, QuantConfig)`` swaps every eligible ``nn.Linear`` (not excluded by name, both
dimensions divisible by 16) for a layer that keeps its master weight in the original dtype and
runs its matmuls in low precision:

* ``mode="fp8"``   e4m3 operands with one scale per 1x128 activation block and per 128x128 weight
                   block, fp32 accumulation (``backend="native"``: the sm_100a kernels in
                   :mod:`forgeminds_b200.ops.quant`).
* ``mode="int8"``  int8 weights and activations with per-row absmax scales, int32 accumulation.
* ``mode="int8_wo"`` int8 weight-only with frozen base weights.

The reference resolves the same modes to Transformer Engine / torchao (``forgemind/quant.py:30-159``);
those backends are still accepted (``backend="te" | "torchao"``) when the libraries are installed.
Without a GPU the native layers run an exact PyTorch emulation of the same quantisation (used by
the CPU tests).
"""
from __future__ import annotations

import contextlib
import functools
import importlib.util

import torch
import torch.nn as nn
import torch.nn.functional as F

from .config import QuantConfig
from .perf import warn_once

__all__ = ["quantize_model", "QuantState", "resolve_backend", "Int8Linear", "Fp8Linear", "make_optimizer_8bit",
           "quantize_rows_int8", "quantize_blocks_fp8"]

FP8_MAX = 448.0          # largest finite e4m3 value


@functools.lru_cache(maxsize=16)
def _installed(name: str) -> bool:
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError):
        return False


def resolve_backend(q: QuantConfig) -> str:
    """``none | native | te | torchao`` for the given config (raises when it cannot be served)."""
    if q.mode == "none":
        return "none"
    if q.mode not in ("fp8", "int8", "int8_wo"):
        raise ValueError(f"unknown quant mode {q.mode!r}")
    if q.backend == "te":
        if not _installed("transformer_engine"):
            raise RuntimeError("backend 'te' requested but transformer_engine is not installed")
        if q.mode != "fp8":
            raise RuntimeError("INT8 is not available through Transformer Engine; use backend 'native' or 'torchao'")
        return "te"
    if q.backend == "torchao":
        if not _installed("torchao"):
            raise RuntimeError("backend 'torchao' requested but torchao is not installed")
        return "torchao"
    if q.backend not in ("auto", "native"):
        raise ValueError(f"unknown quant backend {q.backend!r}")
    return "native"


def _eligible(module, name: str, q: QuantConfig) -> bool:
    return (isinstance(module, nn.Linear) and not any(tag in name for tag in q.exclude)
            and module.in_features % 16 == 0 and module.out_features % 16 == 0)


# ------------------------------------------------------------------------------ quantisers (PyTorch statements)
def quantize_rows_int8(x: torch.Tensor):
    """Per-row symmetric int8: returns ``(q int8 [rows, cols], scale fp32 [rows])`` with
    ``x ~= q * scale[:, None]``."""
    xf = x.float()
    scale = xf.abs().amax(dim=-1).clamp(min=1e-12) / 127.0
    q = torch.round(xf / scale[:, None]).clamp_(-127, 127).to(torch.int8)
    return q, scale


def quantize_blocks_fp8(x: torch.Tensor, block_rows: int, block_cols: int):
    """e4m3 with one fp32 scale per ``block_rows x block_cols`` tile: returns ``(q, scale)`` where
    ``scale`` has shape ``[ceil(rows / block_rows), ceil(cols / block_cols)]``."""
    rows, cols = x.shape
    pr, pc = -rows % block_rows, -cols % block_cols
    xf = F.pad(x.float(), (0, pc, 0, pr))
    tiles = xf.view((rows + pr) // block_rows, block_rows, (cols + pc) // block_cols, block_cols)
    scale = tiles.abs().amax(dim=(1, 3)).clamp(min=1e-12) / FP8_MAX
    q = (tiles / scale[:, None, :, None]).view(rows + pr, cols + pc)[:rows, :cols].to(torch.float8_e4m3fn)
    return q, scale


def _dequant_fp8(q, scale, block_rows, block_cols):
    rows, cols = q.shape
    s = scale.repeat_interleave(block_rows, dim=0)[:rows].repeat_interleave(block_cols, dim=1)[:, :cols]
    return q.float() * s


# ------------------------------------------------------------------------------ layers
class _QuantLinearFn(torch.autograd.Function):
    """Low-precision forward / input-gradient products; the weight gradient uses bf16 operands (its
    reduction runs over tokens, where per-row scales do not factor out)."""

    @staticmethod
    def forward(ctx, x, weight, mode, block):
        ctx.save_for_backward(x, weight)
        ctx.mode, ctx.block = mode, block
        x2 = x.reshape(-1, x.shape[-1])
        y = _qmatmul(x2, weight, mode, block, transpose_w=True)
        return y.view(*x.shape[:-1], weight.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = _qmatmul(dy2, weight, ctx.mode, ctx.block, transpose_w=False).view(x.shape).to(x.dtype)
        if ctx.needs_input_grad[1]:
            x2 = x.reshape(-1, x.shape[-1])
            if x2.is_cuda and x2.dtype == torch.bfloat16:
                from .ops.functional import gemm
                main = getattr(weight, "_fm_main_grad", None)
                if main is not None and dy2.dtype == torch.bfloat16:
                    # a flat parameter store owns this weight: accumulate into its fp32 gradient buffer in place
                    gemm(dy2.contiguous(), x2.contiguous(), a_mn=True, b_mn=True, out=main, c=main, beta=1.0,
                         allow_split=True)
                    dw = None
                else:
                    dw = gemm(dy2.contiguous(), x2.contiguous(), a_mn=True, b_mn=True, out_dtype=torch.float32,
                              allow_split=True).to(weight.dtype)
            else:
                dw = (dy2.float().t() @ x2.float()).to(weight.dtype)
        return dx, dw, None, None


def _qmatmul(a, weight, mode, block, transpose_w):
    """``a @ weight.T`` (``transpose_w``) or ``a @ weight`` with both operands quantised."""
    if a.is_cuda:
        from . import ops
        if ops.available():
            from .ops import quant as qops
            return qops.qmatmul(a, weight, mode, block, transpose_w)
    w = weight.t() if not transpose_w else weight          # [N, K] so that the product is a @ w.T
    if mode == "int8":
        qa, sa = quantize_rows_int8(a)
        qw, sw = quantize_rows_int8(w)
        acc = qa.to(torch.int32) @ qw.to(torch.int32).t() if not a.is_cuda else \
            (qa.float() @ qw.float().t()).to(torch.int32)
        return acc.float() * sa[:, None] * sw[None, :]
    qa, sa = quantize_blocks_fp8(a, 1, block)
    qw, sw = quantize_blocks_fp8(w.contiguous(), block, block)
    return _dequant_fp8(qa, sa, 1, block) @ _dequant_fp8(qw, sw, block, block).t()


class _QuantLinear(nn.Linear):
    mode = "int8"

    def __init__(self, in_features, out_features, bias=True, device=None, dtype=None, block: int = 128):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.block = block

    @classmethod
    def from_linear(cls, lin: nn.Linear, block: int = 128):
        new = cls(lin.in_features, lin.out_features, bias=lin.bias is not None, device=lin.weight.device,
                  dtype=lin.weight.dtype, block=block)
        new.weight = lin.weight
        if lin.bias is not None:
            new.bias = lin.bias
        return new

    def forward(self, x):
        y = _QuantLinearFn.apply(x, self.weight, self.mode, self.block)
        return y if self.bias is None else y + self.bias.to(y.dtype)


class Int8Linear(_QuantLinear):
    mode = "int8"


class Fp8Linear(_QuantLinear):
    mode = "fp8"


class Int8WeightOnlyLinear(nn.Module):
    """Frozen int8 weight with per-output-row scales; activations stay in their dtype."""

    def __init__(self, lin: nn.Linear):
        super().__init__()
        q, s = quantize_rows_int8(lin.weight.detach())
        self.register_buffer("qweight", q)
        self.register_buffer("scale", s)
        self.in_features, self.out_features = lin.in_features, lin.out_features
        self.bias = lin.bias

    def forward(self, x):
        w = (self.qweight.to(x.dtype) * self.scale.to(x.dtype)[:, None])
        return F.linear(x, w, None if self.bias is None else self.bias.to(x.dtype))


class QuantState:
    """Resolved backend plus the autocast context some backends need around the forward pass."""

    def __init__(self, backend, mode, recipe=None, group=None, swapped: int = 0):
        self.backend, self.mode, self.recipe, self.group = backend, mode, recipe, group
        self.swapped = swapped
        self._ctx = None
        if backend == "te":
            import transformer_engine.pytorch as te
            if hasattr(te, "autocast"):
                self._ctx = functools.partial(te.autocast, enabled=True, recipe=recipe)
            else:
                self._ctx = functools.partial(te.fp8_autocast, enabled=True, fp8_recipe=recipe, fp8_group=group)

    def autocast(self):
        return contextlib.nullcontext() if self._ctx is None else self._ctx()


def _swap(model: nn.Module, q: QuantConfig, build) -> int:
    n = 0
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            fqn = f"{parent_name}.{child_name}" if parent_name else child_name
            if _eligible(child, fqn, q) and not isinstance(child, _QuantLinear):
                setattr(parent, child_name, build(child))
                n += 1
    return n


def quantize_model(model: nn.Module, q: QuantConfig, dp_group=None) -> QuantState:
    backend = resolve_backend(q)
    if backend == "none":
        return QuantState("none", "none")
    if backend == "native":
        block = int(getattr(q, "fp8_block", 128))
        if q.mode == "fp8":
            n = _swap(model, q, lambda lin: Fp8Linear.from_linear(lin, block))
        elif q.mode == "int8":
            n = _swap(model, q, lambda lin: Int8Linear.from_linear(lin, block))
        else:
            n = _swap(model, q, Int8WeightOnlyLinear)
        if not n:
            warn_once("quantize_model matched no Linear layer -- check QuantConfig.exclude", key="quant-noop")
        return QuantState("native", q.mode, swapped=n)
    if backend == "te":
        import transformer_engine.pytorch as te
        from transformer_engine.common.recipe import DelayedScaling, Format

        def build(lin):
            new = te.Linear(lin.in_features, lin.out_features, bias=lin.bias is not None,
                            params_dtype=lin.weight.dtype, device=lin.weight.device)
            with torch.no_grad():
                new.weight.copy_(lin.weight)
                if lin.bias is not None:
                    new.bias.copy_(lin.bias)
            return new
        n = _swap(model, q, build)
        recipe = DelayedScaling(fp8_format=Format.HYBRID, amax_history_len=16, amax_compute_algo="max")
        return QuantState("te", "fp8", recipe, dp_group, swapped=n)
    # torchao
    keep = lambda m, fqn: _eligible(m, fqn, q)                      # noqa: E731
    if q.mode == "fp8":
        from torchao.float8 import Float8LinearConfig, convert_to_float8_training
        convert_to_float8_training(model, config=Float8LinearConfig.from_recipe_name("tensorwise"),
                                   module_filter_fn=keep)
    elif q.mode == "int8":
        from torchao.prototype.quantized_training import (Int8MixedPrecisionTrainingConfig,
                                                          int8_mixed_precision_training)
        from torchao.quantization import quantize_
        quantize_(model, int8_mixed_precision_training(Int8MixedPrecisionTrainingConfig()), filter_fn=keep)
    else:
        from torchao.quantization import Int8WeightOnlyConfig, quantize_
        quantize_(model, Int8WeightOnlyConfig(), filter_fn=keep)
        for name, mod in model.named_modules():
            if isinstance(mod, nn.Linear) and _eligible(mod, name, q):
                for p in mod.parameters(recurse=False):
                    p.requires_grad_(False)
    return QuantState("torchao", q.mode)


def make_optimizer_8bit(groups, lr, betas, eps):
    if _installed("torchao"):
        from torchao.optim import AdamW8bit
        return AdamW8bit(groups, lr=lr, betas=betas, eps=eps)
    warn_once("optimizer_8bit needs torchao; using fp32 AdamW states instead", key="adamw8bit")
    return torch.optim.AdamW(groups, lr=lr, betas=betas, eps=eps)
