"""Mixture-of-experts layer on the sm_100a kernels (one GPU; no host read anywhere).

Pipeline for tokens ``x [N, d]`` (bf16):

1. gate logits on the tcgen05 GEMM, then one router kernel: fp32 softmax, top-k, renormalised
   weights, per-expert counts and the sums the auxiliary losses need;
2. a device-side slot plan: every routed entry gets a row in an expert-major buffer whose expert
   regions start on 256-row boundaries (dropless) or have a fixed capacity (overflow dropped);
3. gather -> grouped GEMMs (gate, up) -> SwiGLU -> grouped GEMM (down) -> weighted combine.

The grouped GEMM is the dense tcgen05 kernel with a per-row-tile expert table: the B operand of
each row tile is picked by the z coordinate of a 3-D TMA map over the stacked expert weights. Regions
are aligned to 256 rows so that the products run on CTA pairs (256-row tiles over two SMs, each SM
loading half of the expert's weight tile).
Weight gradients use the "one output per group" mode of the same kernel (reduction over the rows of
each region). The reference does the same work with a sort, ``index_add`` and
``torch._grouped_mm`` / a per-expert loop (``forgemind/moe.py:227-251``).
"""
from __future__ import annotations

import math

import torch
from torch.autograd.function import once_differentiable

from . import require, status_word
from .functional import bf16_of, gemm

BF16 = torch.bfloat16
ALIGN = 256          # rows: expert regions start on multiples of it, so that 256-row tiles never mix experts


class _Route(torch.autograd.Function):
    """logits [N, E] -> (weights fp32 [N, k], idx int32 [N, k], aux scalar)."""

    @staticmethod
    def forward(ctx, logits, k, aux_coef, z_coef):
        C = require()
        n, E = logits.shape
        probs, weights, idx, lse, partial, counts = C.router_fwd(logits, k)
        col = partial.sum(dim=0)                               # [E + 1]: sum of probs per expert, sum of lse^2
        frac = counts.to(torch.float32) / float(n * k)
        aux = E * (frac * (col[:E] / n)).sum()
        z = col[E] / n
        ctx.save_for_backward(probs, idx, weights, lse, frac)
        ctx.coefs = (float(aux_coef), float(z_coef), n, E, logits.dtype)
        ctx.mark_non_differentiable(idx, counts)
        return weights, idx, aux_coef * aux + z_coef * z, counts

    @staticmethod
    @once_differentiable
    def backward(ctx, dweights, _didx, daux, _dcounts):
        C = require()
        probs, idx, weights, lse, frac = ctx.saved_tensors
        aux_coef, z_coef, n, E, dtype = ctx.coefs
        aux_grad = zc = None
        if daux is not None:
            g = daux.to(torch.float32)
            aux_grad = (g * (aux_coef * E / n) * frac).contiguous()
            zc = (g * (z_coef * 2.0 / n)).reshape(1).contiguous()
        dw = dweights.to(torch.float32).contiguous() if dweights is not None else None
        return C.router_bwd(probs, idx, weights, lse, dw, aux_grad, zc, dtype), None, None, None


class _Experts(torch.autograd.Function):
    """Gather, SwiGLU experts, weighted combine for an already planned routing.

    ``limit`` (device int, first row past the last expert's region) is given for dropless plans: every row
    tile below it belongs to an expert and is written whole by the grouped products (padding rows of the
    gathered input are zero, so theirs are too), and nothing below reads a row at or past it, so the
    buffers need no clearing. With a capacity an unused tile inside a region would feed stale values into
    the expert weight gradients: those (bounded) buffers are cleared."""

    @staticmethod
    def forward(ctx, x, route_w, w1, w3, w2, slot_of, token_of, region, tile_group, k, limit=None):
        C = require()
        st = status_word(x.device)
        n, d = x.shape
        S = token_of.numel()
        h = w1.shape[2]
        alloc = torch.empty if limit is not None else torch.zeros
        b1, b3, b2 = bf16_of(w1), bf16_of(w3), bf16_of(w2)
        xs = C.moe_gather(x, token_of)
        gu = alloc((S, 2 * h), dtype=BF16, device=x.device)
        C.gemm_grouped_rows(xs, b1, gu[:, :h], tile_group, True, False, st, True)
        C.gemm_grouped_rows(xs, b3, gu[:, h:], tile_group, True, False, st, True)
        act = C.swiglu_fwd(gu[:, :h], gu[:, h:], limit)
        ys = alloc((S, d), dtype=BF16, device=x.device)
        C.gemm_grouped_rows(act, b2, ys, tile_group, True, False, st, True)
        rw = route_w.detach().to(torch.float32).contiguous()
        out = C.moe_combine(ys, slot_of, rw, n, k)
        ctx.save_for_backward(xs, gu, ys, rw, slot_of, region, tile_group, b1, b3, b2, limit)
        ctx.params = (w1, w3, w2)
        ctx.dims = (n, d, h, k, route_w.dtype)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, dout):
        C = require()
        xs, gu, ys, rw, slot_of, region, tile_group, b1, b3, b2, limit = ctx.saved_tensors
        w1, w3, w2 = ctx.params
        n, d, h, k, rw_dtype = ctx.dims
        st = status_word(dout.device)
        S = xs.shape[0]
        alloc = torch.empty if limit is not None else torch.zeros
        dout = dout.contiguous()
        dys, drw = C.moe_combine_bwd(dout, ys, slot_of, rw, k)                # zero in rows that hold no entry
        act = C.swiglu_fwd(gu[:, :h], gu[:, h:], limit)                       # recomputed
        grads = {}

        def wgrad(name, param, a, b):
            main = getattr(param, "_fm_main_grad", None)
            if main is not None:
                C.gemm_grouped_wgrad(a, b, main, region, True, st)
                grads[name] = None
            else:
                g = torch.empty(param.shape, dtype=torch.float32, device=dout.device)
                C.gemm_grouped_wgrad(a, b, g, region, False, st)
                grads[name] = g if g.dtype == param.dtype else g.to(param.dtype)

        wgrad("w2", w2, act, dys)
        dact = alloc((S, h), dtype=BF16, device=dout.device)
        C.gemm_grouped_rows(dys, b2, dact, tile_group, False, False, st, True)    # dys @ w2[e]^T
        dgu = alloc(gu.shape, dtype=BF16, device=dout.device)
        C.swiglu_bwd(gu[:, :h], gu[:, h:], dact, dgu[:, :h], dgu[:, h:], limit)
        wgrad("w1", w1, xs, dgu[:, :h])
        wgrad("w3", w3, xs, dgu[:, h:])
        dxs = alloc((S, d), dtype=BF16, device=dout.device)
        C.gemm_grouped_rows(dgu[:, :h], b1, dxs, tile_group, False, False, st, True)
        C.gemm_grouped_rows(dgu[:, h:], b3, dxs, tile_group, False, True, st, True)
        dx = C.moe_combine(dxs, slot_of, None, n, k)
        return dx, drw.view(n, k).to(rw_dtype), grads["w1"], grads["w3"], grads["w2"], None, None, None, None, None, None


def plan(idx, n_experts: int, capacity: int = 0):
    """Slot plan for ``idx [N, k]`` (int32): ``(slot_of_entry, token_of_slot, region, tile_group, limit)``.
    ``capacity > 0`` gives every expert a fixed region of ``ceil256(capacity)`` rows (``limit`` is None);
    a dropless plan also returns ``limit``, a device int holding the first row past the last region."""
    C = require()
    n, k = idx.shape
    if capacity > 0:
        cap = (capacity + ALIGN - 1) // ALIGN * ALIGN
        slots = n_experts * cap
        slot_of, token_of, region, _ = C.moe_plan(idx, n_experts, ALIGN, cap, 1, slots)
        limit = None
    else:
        # one more (always empty) expert: its region starts where the live rows end
        slots = (n * k + ALIGN - 1) // ALIGN * ALIGN + (n_experts + 1) * ALIGN
        slot_of, token_of, region, _ = C.moe_plan(idx, n_experts + 1, ALIGN, 0, 0, slots)
        limit, region = region[n_experts], region[:n_experts]
    tile_group = C.moe_tile_groups(region, slots // 128)
    return slot_of, token_of, region, tile_group, limit


def moe_forward_native(moe, x):
    """``x [N, d]`` bf16 -> MoE output ``[N, d]``; sets ``moe.last_aux``."""
    from .functional import linear
    if moe.ep_size > 1:
        if moe.ep_engine is None:
            raise RuntimeError("expert parallelism on the native path needs parallel.ep.attach(model, ctx)")
        return moe.ep_engine.forward(moe, x)
    gate = moe.router.gate.weight
    if gate.shape[0] % 8 == 0:
        logits = linear(x, gate)
    else:       # the GEMM epilogue stores 16-byte vectors: an odd expert count takes the library matmul
        logits = torch.nn.functional.linear(x, gate.to(x.dtype))
    route_w, idx, aux, _counts = _Route.apply(logits, moe.top_k, moe.aux_coef, moe.z_coef)
    moe.last_aux = aux
    slot_of, token_of, region, tile_group, limit = plan(idx, moe.n_experts, moe.capacity(x.shape[0]))
    ex = moe.experts
    out = _Experts.apply(x, route_w, ex.w1, ex.w3, ex.w2, slot_of, token_of, region, tile_group, moe.top_k, limit)
    if moe.shared is not None:
        from .functional import linear_multi, swiglu_linear
        gu = linear_multi(x, (moe.shared.w1.weight, moe.shared.w3.weight))
        out = swiglu_linear(gu, moe.shared.w2.weight, out)
    return out
