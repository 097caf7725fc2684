"""Autograd wrappers around the native kernels (GPU only; callers pick the torch path on CPU).

Conventions
-----------
* Activations are bf16, 2-D ``[tokens, features]`` inside these functions.
* ``linear`` computes ``x @ W.T`` with ``W`` in ``nn.Linear`` layout. The weight may be an fp32
  master parameter: a bf16 shadow copy is cached on the parameter (``_fm_shadow``) and refreshed
  only when the parameter's version changed, instead of being re-cast on every forward.
* Weight gradients are produced in fp32 by the GEMM epilogue. If the parameter carries a
  ``_fm_main_grad`` buffer, the weight-gradient GEMM accumulates straight into it (no separate
  add pass) and autograd receives ``None`` for that parameter.
"""
from __future__ import annotations

import math

import torch
from torch.autograd.function import once_differentiable

from . import require, status_word

BF16 = torch.bfloat16


# ------------------------------------------------------------------------------ helpers
_weights_epoch = 0


def _optimizer_stepped(*_args, **_kw) -> None:
    global _weights_epoch
    _weights_epoch += 1


# torch's fused optimizers update parameters without touching their version counters, so a cached
# bf16 copy cannot rely on ``_version`` alone: every optimizer step (of any optimizer) starts a new epoch.
from torch.optim.optimizer import register_optimizer_step_post_hook as _register_step_hook  # noqa: E402

_register_step_hook(_optimizer_stepped)


def bf16_of(p: torch.Tensor) -> torch.Tensor:
    """bf16 view of a parameter: itself when already bf16, else a cached shadow copy.

    A cache entry is ``(shadow, version)`` when a flat store owns the shadow and keeps it current
    itself, or ``(shadow, version, epoch)`` when it was made here; the latter is refreshed when the
    parameter's version changed or any optimizer has stepped since."""
    if hasattr(p, "to_local"):
        raise TypeError("the sm_100a kernels take plain tensors; got a DTensor parameter (sharded by FSDP2 / DTensor "
                        "tensor parallelism). Call the module through its wrapper or switch the block to native=False")
    if p.dtype == BF16:
        return p.detach()
    cached = getattr(p, "_fm_shadow", None)
    if cached is not None and cached[0].device == p.device and cached[0].shape == p.shape:
        if cached[1] == p._version and (len(cached) == 2 or cached[2] == _weights_epoch):
            return cached[0]
        shadow = cached[0]          # refresh in place: the buffer may be a view owned by a flat store
        managed = len(cached) == 2
    else:
        shadow = torch.empty(p.shape, dtype=BF16, device=p.device)
        managed = False
    src = p.detach()
    if src.dtype == torch.float32 and src.is_contiguous():
        require().scale_cast(src, shadow, 1.0)
    else:
        shadow.copy_(src)
    try:
        p._fm_shadow = (shadow, p._version) if managed else (shadow, p._version, _weights_epoch)
    except Exception:
        pass
    return shadow


def gemm(a, b, *, a_mn=False, b_mn=False, out=None, c=None, alpha=1.0, beta=0.0, alpha_dev=None,
         out_dtype=BF16, allow_split=False, force_bn=0):
    """``out = alpha * A' @ B'.T + beta * c`` where ``A'`` is ``a`` ([M,K]) or ``a.T`` when
    ``a_mn`` (``a`` stored [K,M]); likewise for ``b`` ([N,K] or [K,N])."""
    C = require()
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    C.gemm(a, b, out, c, a_mn, b_mn, float(alpha), float(beta), alpha_dev, allow_split, status_word(a.device),
           int(force_bn))
    return out


def _rows(x):
    return x.reshape(-1, x.shape[-1])


def _gemm_like(x, x2, w, **kw):
    """``x2 @ w.T`` written into a freshly allocated tensor shaped like ``x`` with the last dim
    replaced (the autograd output is then an owning tensor, not a view, and may be updated in place)."""
    y = torch.empty((*x.shape[:-1], w.shape[0]), dtype=BF16, device=x.device)
    gemm(x2, w, out=y.view(-1, w.shape[0]), **kw)
    return y


# ------------------------------------------------------------------------------ linear
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual):
        w = bf16_of(weight)
        x2 = _rows(x)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        res2 = None
        if residual is not None:
            res2 = _rows(residual)
            if not res2.is_contiguous():
                res2 = res2.contiguous()
        y = _gemm_like(x, x2, w, c=res2, beta=1.0 if res2 is not None else 0.0)
        ctx.save_for_backward(x2, w)
        ctx.weight = weight
        ctx.x_shape = x.shape
        ctx.has_res = residual is not None
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        weight = ctx.weight
        dy2 = _rows(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "_fm_main_grad", None)
            if main is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main, c=main, beta=1.0, allow_split=True)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32, allow_split=True)
                if dw.dtype != weight.dtype:
                    dw = dw.to(weight.dtype)
        return dx, dw, (dy if ctx.has_res else None)


def linear(x, weight, residual=None):
    """``x @ weight.T (+ residual)`` on the tcgen05 GEMM; the residual add runs in the epilogue."""
    return _Linear.apply(x, weight, residual)


def _adjacent(views) -> bool:
    """True when the tensors are contiguous row blocks lying back to back in one storage."""
    nxt = base = None
    for v in views:
        if v is None or not v.is_contiguous():
            return False
        store = v.untyped_storage().data_ptr()
        if base is None:
            base = store
        if store != base:                  # neighbours by accident of the allocator do not count
            return False
        if nxt is not None and v.data_ptr() != nxt:
            return False
        nxt = v.data_ptr() + v.numel() * v.element_size()
    return True


def _stack_view(views):
    """Zero-copy ``[sum rows, K]`` view over adjacent row blocks."""
    first = views[0]
    rows = sum(v.shape[0] for v in views)
    return torch.as_strided(first, (rows, first.shape[1]), (first.shape[1], 1))


def fused_bf16(weights) -> torch.Tensor:
    """bf16 ``[sum N_i, K]`` matrix of several ``[N_i, K]`` weights. No copy when their shadows are
    neighbours in memory (the flat parameter store lays them out that way); otherwise the
    concatenation is cached on the first weight until any of the versions changes."""
    shadows = [bf16_of(w) for w in weights]
    if len(shadows) == 1:
        return shadows[0]
    if _adjacent(shadows):
        return _stack_view(shadows)
    head = weights[0]
    key = (_weights_epoch,) + tuple((id(w), w._version) for w in weights)
    cached = getattr(head, "_fm_fused", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    fused = torch.cat(shadows, dim=0)
    head._fm_fused = (key, fused)
    return fused


def fused_main_grad(weights):
    grads = [getattr(w, "_fm_main_grad", None) for w in weights]
    if any(g is None for g in grads):
        return None
    if len(grads) == 1:
        return grads[0]
    return _stack_view(grads) if _adjacent(grads) else None


class _LinearMulti(torch.autograd.Function):
    """``x @ cat(weights).T`` as one GEMM (fused q|k|v or gate|up projection) while the weights
    stay separate parameters."""

    @staticmethod
    def forward(ctx, x, *weights):
        w = fused_bf16(weights)
        x2 = _rows(x)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = _gemm_like(x, x2, w)
        ctx.save_for_backward(x2, w)
        ctx.weights = weights
        ctx.x_shape = x.shape
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        weights = ctx.weights
        dy2 = _rows(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = gemm(dy2, w, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        grads = [None] * len(weights)
        if any(ctx.needs_input_grad[1:]):
            main = fused_main_grad(weights)
            if main is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main, c=main, beta=1.0, allow_split=True)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32, allow_split=True)
                lo = 0
                for i, wt in enumerate(weights):
                    piece = dw[lo: lo + wt.shape[0]]
                    lo += wt.shape[0]
                    own = getattr(wt, "_fm_main_grad", None)
                    if own is not None:
                        own.add_(piece)
                    elif ctx.needs_input_grad[1 + i]:
                        grads[i] = piece if piece.dtype == wt.dtype else piece.to(wt.dtype)
        return (dx, *grads)


def linear_multi(x, weights):
    return _LinearMulti.apply(x, *weights)


def _weight_grads(ctx_needs, weights, dy2, x2):
    """Weight gradient of a (fused) projection: accumulate into main-grad buffers when the
    parameters carry them, otherwise hand fp32 slices back to autograd."""
    grads = [None] * len(weights)
    if not any(ctx_needs):
        return grads
    main = fused_main_grad(weights)
    if main is not None:
        gemm(dy2, x2, a_mn=True, b_mn=True, out=main, c=main, beta=1.0, allow_split=True)
        return grads
    dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32, allow_split=True)
    lo = 0
    for i, wt in enumerate(weights):
        piece = dw[lo: lo + wt.shape[0]]
        lo += wt.shape[0]
        own = getattr(wt, "_fm_main_grad", None)
        if own is not None:
            own.add_(piece)
        elif ctx_needs[i]:
            grads[i] = piece if piece.dtype == wt.dtype else piece.to(wt.dtype)
    return grads


def _norm_acc(ctx):
    """fp32 gradient buffer of the norm weight when a flat store owns it and it wants a gradient: the column
    sum of the RMSNorm backward then adds into it, and autograd gets no tensor to accumulate."""
    main = getattr(ctx, "norm_main", None)
    if main is None or not ctx.needs_input_grad[1] or main.dtype != torch.float32 or not main.is_contiguous():
        return None
    return main


class _NormLinearMulti(torch.autograd.Function):
    """``rms_norm(x) @ cat(weights).T``. Only ``x`` and the per-row ``rstd`` are kept; the normalised
    activations are recomputed in the backward (one extra pass over ``x`` instead of a saved tensor).

    With ``passthrough`` the Function also returns ``x`` itself as a second output. A block uses that
    output for its residual connection, so the gradient of the residual stream arrives here and is
    added inside the RMSNorm backward kernel instead of by a separate elementwise add."""

    @staticmethod
    def forward(ctx, x, norm_w, eps, passthrough, *weights):
        C = require()
        w = fused_bf16(weights)
        x2 = _rows(x)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        nw = norm_w.detach()
        if nw.dtype not in (torch.float32, x2.dtype):
            nw = nw.to(x2.dtype)
        nw = nw.contiguous()
        h, rstd = C.rmsnorm_fwd(x2, nw, eps)
        y = _gemm_like(x, h, w)
        ctx.save_for_backward(x2, nw, rstd, w)
        ctx.weights, ctx.eps, ctx.x_shape, ctx.nw_dtype = weights, eps, x.shape, norm_w.dtype
        ctx.norm_main = getattr(norm_w, "_fm_main_grad", None)      # a flat gradient store owns the norm weight
        if passthrough:
            return y, x.view_as(x)
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, dy, dres=None):
        C = require()
        x2, nw, rstd, w = ctx.saved_tensors
        dy2 = _rows(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        h, _ = C.rmsnorm_fwd(x2, nw, ctx.eps)                       # recompute
        grads = _weight_grads(ctx.needs_input_grad[4:], ctx.weights, dy2, h)
        dx = dnw = None
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            dh = gemm(dy2, w, b_mn=True)
            if dres is not None:
                dres = _rows(dres)
                if dres.dtype != dh.dtype:
                    dres = dres.to(dh.dtype)
                if not dres.is_contiguous():
                    dres = dres.contiguous()
            dx, dnw = C.rmsnorm_bwd(dh, x2, nw, rstd, dres, ctx.needs_input_grad[1], _norm_acc(ctx))
            dx = dx.view(ctx.x_shape)
            if dnw is not None and dnw.dtype != ctx.nw_dtype:
                dnw = dnw.to(ctx.nw_dtype)
        elif dres is not None:
            dx = dres
        return (dx, dnw, None, None, *grads)


def norm_linear_multi(x, norm_w, eps, weights, passthrough: bool = False):
    """``passthrough=True`` returns ``(y, x)``: use the returned ``x`` for the residual connection."""
    return _NormLinearMulti.apply(x, norm_w, eps, passthrough, *weights)


class _SwiGLULinear(torch.autograd.Function):
    """``(silu(gate) * up) @ W.T + residual`` from the fused gate|up projection output. Only ``gu``
    is kept; the activation is recomputed in the backward."""

    @staticmethod
    def forward(ctx, gu, weight, residual):
        C = require()
        w = bf16_of(weight)
        g2 = _rows(gu)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        h = g2.shape[1] // 2
        act = C.swiglu_fwd(g2[:, :h], g2[:, h:])
        res2 = None
        if residual is not None:
            res2 = _rows(residual)
            if not res2.is_contiguous():
                res2 = res2.contiguous()
        y = _gemm_like(gu, act, w, c=res2, beta=1.0 if res2 is not None else 0.0)
        ctx.save_for_backward(g2, w)
        ctx.weight, ctx.gu_shape, ctx.has_res = weight, gu.shape, residual is not None
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, dy):
        C = require()
        g2, w = ctx.saved_tensors
        h = g2.shape[1] // 2
        dy2 = _rows(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        act = C.swiglu_fwd(g2[:, :h], g2[:, h:])                     # recompute
        (dw,) = _weight_grads(ctx.needs_input_grad[1:2], (ctx.weight,), dy2, act)
        dgu = None
        if ctx.needs_input_grad[0]:
            dact = gemm(dy2, w, b_mn=True)
            dgu = torch.empty_like(g2)
            C.swiglu_bwd(g2[:, :h], g2[:, h:], dact, dgu[:, :h], dgu[:, h:])
            dgu = dgu.view(ctx.gu_shape)
        return dgu, dw, (dy if ctx.has_res else None)


def swiglu_linear(gu, weight, residual=None):
    return _SwiGLULinear.apply(gu, weight, residual)


class _Embedding(torch.autograd.Function):
    """Row gather from the bf16 shadow of an fp32 table; the gradient is scattered in fp32."""

    @staticmethod
    def forward(ctx, tokens, weight):
        table = bf16_of(weight)
        ctx.save_for_backward(tokens)
        ctx.weight = weight
        return torch.nn.functional.embedding(tokens, table)

    @staticmethod
    @once_differentiable
    def backward(ctx, dy):
        (tokens,) = ctx.saved_tensors
        weight = ctx.weight
        flat = tokens.reshape(-1)
        rows = dy.reshape(-1, dy.shape[-1]).to(torch.float32)
        main = getattr(weight, "_fm_main_grad", None)
        if main is not None:
            main.index_add_(0, flat, rows)
            return None, None
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=dy.device).index_add_(0, flat, rows)
        return None, dw if dw.dtype == weight.dtype else dw.to(weight.dtype)


def embedding(tokens, weight):
    return _Embedding.apply(tokens, weight)


# ------------------------------------------------------------------------------ RMSNorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        C = require()
        x2 = _rows(x).contiguous()
        wd = w.detach()
        if wd.dtype not in (torch.float32, x2.dtype):
            wd = wd.to(x2.dtype)
        y, rstd = C.rmsnorm_fwd(x2, wd.contiguous(), eps)
        ctx.save_for_backward(x2, wd, rstd)
        ctx.w_dtype = w.dtype
        return y.view(x.shape)

    @staticmethod
    @once_differentiable
    def backward(ctx, dy):
        C = require()
        x2, wd, rstd = ctx.saved_tensors
        dx, dw = C.rmsnorm_bwd(_rows(dy).contiguous(), x2, wd, rstd, None, ctx.needs_input_grad[1])
        if dw is not None and dw.dtype != ctx.w_dtype:
            dw = dw.to(ctx.w_dtype)
        return dx.view(dy.shape), dw, None


def rms_norm(x, w, eps=1e-6):
    return _RMSNorm.apply(x, w, eps)


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, w, eps):
        C = require()
        x2, d2 = _rows(x).contiguous(), _rows(delta).contiguous()
        wd = w.detach()
        if wd.dtype not in (torch.float32, x2.dtype):
            wd = wd.to(x2.dtype)
        xn, y, rstd = C.add_rmsnorm_fwd(x2, d2, wd.contiguous(), eps)
        ctx.save_for_backward(xn, wd, rstd)
        ctx.w_dtype = w.dtype
        return xn.view(x.shape), y.view(x.shape)

    @staticmethod
    @once_differentiable
    def backward(ctx, gxn, gy):
        C = require()
        xn, wd, rstd = ctx.saved_tensors
        gy2 = _rows(gy).contiguous() if gy is not None else torch.zeros_like(xn)
        res = _rows(gxn).contiguous() if gxn is not None else None
        dx, dw = C.rmsnorm_bwd(gy2, xn, wd, rstd, res, ctx.needs_input_grad[2])
        if dw is not None and dw.dtype != ctx.w_dtype:
            dw = dw.to(ctx.w_dtype)
        dx = dx.view(gy.shape if gy is not None else gxn.shape)
        return dx, dx, dw, None


def add_rms_norm(x, delta, w, eps=1e-6):
    """Returns ``(x + delta, rms_norm(x + delta) * w)`` from one pass over the row."""
    return _AddRMSNorm.apply(x, delta, w, eps)


# ------------------------------------------------------------------------------ SwiGLU
class _SwiGLUSplit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        C = require()
        g2 = _rows(gu)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        h = g2.shape[1] // 2
        out = C.swiglu_fwd(g2[:, :h], g2[:, h:])
        ctx.save_for_backward(g2)
        return out.view(*gu.shape[:-1], h)

    @staticmethod
    @once_differentiable
    def backward(ctx, dy):
        C = require()
        (g2,) = ctx.saved_tensors
        h = g2.shape[1] // 2
        dgu = torch.empty_like(g2)
        C.swiglu_bwd(g2[:, :h], g2[:, h:], _rows(dy).contiguous(), dgu[:, :h], dgu[:, h:])
        return dgu.view(*dy.shape[:-1], 2 * h)


def swiglu_split(gu):
    """``silu(gu[..., :h]) * gu[..., h:]``"""
    return _SwiGLUSplit.apply(gu)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        C = require()
        g2, u2 = _rows(gate).contiguous(), _rows(up).contiguous()
        out = C.swiglu_fwd(g2, u2)
        ctx.save_for_backward(g2, u2)
        return out.view(gate.shape)

    @staticmethod
    @once_differentiable
    def backward(ctx, dy):
        C = require()
        g2, u2 = ctx.saved_tensors
        dg, du = torch.empty_like(g2), torch.empty_like(u2)
        C.swiglu_bwd(g2, u2, _rows(dy).contiguous(), dg, du)
        return dg.view(dy.shape), du.view(dy.shape)


def swiglu(gate, up):
    return _SwiGLU.apply(gate, up)


# ------------------------------------------------------------------------------ RoPE on a fused qkv buffer
class _RopeQKV(torch.autograd.Function):
    """Rotates the q and k heads of ``qkv [B, T, (Hq + 2 Hkv) * hd]`` in place (v untouched)."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, n_q, n_kv, hd):
        C = require()
        B, T = qkv.shape[0], qkv.shape[1]
        C.rope(qkv, qkv, cos, sin, T, n_q + n_kv, n_q + 2 * n_kv, hd, 1.0)
        ctx.mark_dirty(qkv)
        ctx.save_for_backward(cos, sin)
        ctx.dims = (T, n_q, n_kv, hd)
        return qkv

    @staticmethod
    @once_differentiable
    def backward(ctx, g):
        C = require()
        cos, sin = ctx.saved_tensors
        T, n_q, n_kv, hd = ctx.dims
        g = g.contiguous()
        out = torch.empty_like(g)           # the incoming gradient is not ours to overwrite
        C.rope(g, out, cos, sin, T, n_q + n_kv, n_q + 2 * n_kv, hd, -1.0)
        return out, None, None, None, None, None


def rope_qkv_(qkv, cos, sin, n_q, n_kv, hd):
    return _RopeQKV.apply(qkv, cos, sin, n_q, n_kv, hd)


# ------------------------------------------------------------------------------ attention
class _Attention(torch.autograd.Function):
    """Causal GQA attention on a fused q|k|v buffer. With ``cos`` / ``sin`` the q and k heads are rotated in
    place first (the buffer comes back as a second, dirty output) and the backward rotates the gradient
    back in the pass that converts the kernel's fp32 dQ sum to bf16. The buffer is ``[B, T, W]`` or, with
    ``bt = (B, T)``, the ``[B * T, W]`` rows of a projection output (autograd lets a Function with two
    outputs modify an input in place only if that input is not a view, so such rows are passed as they are)."""

    @staticmethod
    def forward(ctx, given, n_q, n_kv, hd, causal, cos=None, sin=None, bt=None):
        C = require()
        qkv = given.view(bt[0], bt[1], -1) if given.dim() == 2 else given
        B, T, _ = qkv.shape
        ctx.rope = cos is not None
        if ctx.rope:
            C.rope(qkv, qkv, cos, sin, T, n_q + n_kv, n_q + 2 * n_kv, hd, 1.0)
            ctx.mark_dirty(given)
            ctx.set_materialize_grads(False)
        q = qkv[..., : n_q * hd].unflatten(-1, (n_q, hd))
        k = qkv[..., n_q * hd: (n_q + n_kv) * hd].unflatten(-1, (n_kv, hd))
        v = qkv[..., (n_q + n_kv) * hd:].unflatten(-1, (n_kv, hd))
        o, lse = C.attn_fwd(q, k, v, 1.0 / math.sqrt(hd), causal, status_word(qkv.device))
        if ctx.rope:
            ctx.save_for_backward(given, o, lse, cos, sin)
        else:
            ctx.save_for_backward(given, o, lse)
        ctx.dims = (n_q, n_kv, hd, causal, B, T)
        out = o.view(B, T, n_q * hd)
        return (out, given) if ctx.rope else out

    @staticmethod
    @once_differentiable
    def backward(ctx, d_o, g_qkv=None):
        C = require()
        cos = sin = None
        if ctx.rope:
            given, o, lse, cos, sin = ctx.saved_tensors
            if g_qkv is not None:
                raise RuntimeError("the rotated qkv buffer returned by attention_qkv is not differentiable")
            if d_o is None:
                return (None,) * 8
        else:
            given, o, lse = ctx.saved_tensors
        n_q, n_kv, hd, causal, B, T = ctx.dims
        qkv = given.view(B, T, -1)
        dqkv = torch.empty_like(qkv)
        q = qkv[..., : n_q * hd].unflatten(-1, (n_q, hd))
        k = qkv[..., n_q * hd: (n_q + n_kv) * hd].unflatten(-1, (n_kv, hd))
        v = qkv[..., (n_q + n_kv) * hd:].unflatten(-1, (n_kv, hd))
        dq = dqkv[..., : n_q * hd].unflatten(-1, (n_q, hd))
        dk = dqkv[..., n_q * hd: (n_q + n_kv) * hd].unflatten(-1, (n_kv, hd))
        dv = dqkv[..., (n_q + n_kv) * hd:].unflatten(-1, (n_kv, hd))
        d_o4 = d_o.contiguous().view(B, T, n_q, hd)
        scale, st = 1.0 / math.sqrt(hd), status_word(qkv.device)
        if ctx.rope:
            dq32 = C.attn_bwd(q, k, v, o, d_o4, lse, None, dk, dv, scale, causal, st, None)
            C.rope(dqkv, dqkv, cos, sin, T, n_q + n_kv, n_q + 2 * n_kv, hd, -1.0, dq32)
        else:
            C.attn_bwd(q, k, v, o, d_o4, lse, dq, dk, dv, scale, causal, st, None)
        return dqkv.view(given.shape), None, None, None, None, None, None, None


class _AttentionProj(torch.autograd.Function):
    """``attention(qkv) @ Wo.T + residual`` as one autograd node. In the backward, the product that
    yields ``dO = dY @ Wo`` also emits ``delta = rowsum(dO * O)`` per head from its epilogue, so the
    attention backward needs no separate pass over ``O`` and ``dO``.

    With ``cos`` / ``sin`` the q and k heads of ``qkv`` are first rotated in place (RoPE), and the backward
    rotates the gradient back in the same pass that converts the fp32 dQ sum of the attention kernel to
    bf16, so that sum is read once and no separate conversion kernel runs. ``qkv`` then comes back as a
    second (dirty) output."""

    @staticmethod
    def forward(ctx, qkv, weight, residual, n_q, n_kv, hd, causal, cos=None, sin=None):
        C = require()
        B, T, _ = qkv.shape
        ctx.rope = cos is not None
        if ctx.rope:
            C.rope(qkv, qkv, cos, sin, T, n_q + n_kv, n_q + 2 * n_kv, hd, 1.0)
            ctx.mark_dirty(qkv)
            ctx.set_materialize_grads(False)
        q = qkv[..., : n_q * hd].unflatten(-1, (n_q, hd))
        k = qkv[..., n_q * hd: (n_q + n_kv) * hd].unflatten(-1, (n_kv, hd))
        v = qkv[..., (n_q + n_kv) * hd:].unflatten(-1, (n_kv, hd))
        o, lse = C.attn_fwd(q, k, v, 1.0 / math.sqrt(hd), causal, status_word(qkv.device))
        w = bf16_of(weight)
        o2 = o.view(B * T, n_q * hd)
        res2 = None
        if residual is not None:
            res2 = _rows(residual)
            if not res2.is_contiguous():
                res2 = res2.contiguous()
        y = torch.empty((B, T, w.shape[0]), dtype=BF16, device=qkv.device)
        gemm(o2, w, out=y.view(B * T, w.shape[0]), c=res2, beta=1.0 if res2 is not None else 0.0)
        if ctx.rope:
            ctx.save_for_backward(qkv, o, lse, w, cos, sin)
        else:
            ctx.save_for_backward(qkv, o, lse, w)
        ctx.weight = weight
        ctx.dims = (n_q, n_kv, hd, causal, residual is not None)
        return (y, qkv) if ctx.rope else y

    @staticmethod
    @once_differentiable
    def backward(ctx, dy, g_qkv=None):
        C = require()
        cos = sin = None
        if ctx.rope:
            qkv, o, lse, w, cos, sin = ctx.saved_tensors
            if g_qkv is not None:
                raise RuntimeError("the rotated qkv buffer returned by attention_proj is not differentiable")
            if dy is None:
                return (None,) * 9
        else:
            qkv, o, lse, w = ctx.saved_tensors
        weight = ctx.weight
        n_q, n_kv, hd, causal, has_res = ctx.dims
        B, T, _ = qkv.shape
        st = status_word(qkv.device)
        dy2 = _rows(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        o2 = o.view(B * T, n_q * hd)
        dw = None
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "_fm_main_grad", None)
            if main is not None:
                gemm(dy2, o2, a_mn=True, b_mn=True, out=main, c=main, beta=1.0, allow_split=True)
            else:
                dw = gemm(dy2, o2, a_mn=True, b_mn=True, out_dtype=torch.float32, allow_split=True)
                if dw.dtype != weight.dtype:
                    dw = dw.to(weight.dtype)
        dqkv = None
        if ctx.needs_input_grad[0]:
            d_o = torch.empty_like(o2)
            delta = None
            if hd % 32 == 0 and 256 % hd == 0:
                delta = torch.empty((B, n_q, T), dtype=torch.float32, device=qkv.device)
                C.gemm_rowdot(dy2, w, True, d_o, o2, delta, hd, T, st)
            else:
                gemm(dy2, w, b_mn=True, out=d_o)
            dqkv = torch.empty_like(qkv)
            q = qkv[..., : n_q * hd].unflatten(-1, (n_q, hd))
            k = qkv[..., n_q * hd: (n_q + n_kv) * hd].unflatten(-1, (n_kv, hd))
            v = qkv[..., (n_q + n_kv) * hd:].unflatten(-1, (n_kv, hd))
            dq = dqkv[..., : n_q * hd].unflatten(-1, (n_q, hd))
            dk = dqkv[..., n_q * hd: (n_q + n_kv) * hd].unflatten(-1, (n_kv, hd))
            dv = dqkv[..., (n_q + n_kv) * hd:].unflatten(-1, (n_kv, hd))
            if ctx.rope:
                dq32 = C.attn_bwd(q, k, v, o, d_o.view(B, T, n_q, hd), lse, None, dk, dv, 1.0 / math.sqrt(hd), causal,
                                  st, delta)
                C.rope(dqkv, dqkv, cos, sin, T, n_q + n_kv, n_q + 2 * n_kv, hd, -1.0, dq32)
            else:
                C.attn_bwd(q, k, v, o, d_o.view(B, T, n_q, hd), lse, dq, dk, dv, 1.0 / math.sqrt(hd), causal, st, delta)
        return dqkv, dw, (dy if has_res else None), None, None, None, None, None, None


def attention_proj(qkv, weight, residual, n_q, n_kv, hd, causal=True, rope=None):
    """Causal GQA attention on a fused q|k|v buffer followed by the output projection (+ residual).
    ``rope=(cos, sin)`` rotates the q and k heads of ``qkv`` in place first."""
    if rope is None:
        return _AttentionProj.apply(qkv, weight, residual, n_q, n_kv, hd, causal)
    if qkv._is_view():          # a view cannot be rotated in place by a node with two outputs: rotate it on its own
        return _AttentionProj.apply(rope_qkv_(qkv, rope[0], rope[1], n_q, n_kv, hd), weight, residual, n_q, n_kv, hd,
                                    causal)
    return _AttentionProj.apply(qkv, weight, residual, n_q, n_kv, hd, causal, rope[0], rope[1])[0]


# Whether the SwiGLU runs in the epilogue of the neighbouring product (forward: gate|up product; backward:
# activation-gradient product) or as its own kernel. Measured on a B200 at M = 8192, d = 1024, h = 2816
# (norm + MLP forward + backward, cold L2): forward fused 0.487 ms against 0.507 ms unfused (forward alone
# 0.122 against 0.146), since the gate|up product runs on CTA pairs with its TMEM reads one chunk pair
# ahead of 32-byte stores. The backward form is still slower (0.543 ms with both fused): its epilogue
# reads gate|up and writes two outputs per accumulator chunk. Both forms are tested.
MLP_FUSE_FWD = True
MLP_FUSE_BWD = False


class _MLPBlock(torch.autograd.Function):
    """``x + W2 (silu(W1 n) * (W3 n))`` with ``n = rms_norm(x)``, the SwiGLU fused into GEMM epilogues.

    Forward: the gate|up product writes gate, up and the activation from its epilogue. Backward: the
    product ``dY @ W2`` turns its accumulator (the activation gradient) straight into the gate and up
    gradients in its epilogue. Kept for the backward: ``x``, ``rstd``, gate|up (the normalised input
    and the activation are recomputed)."""

    @staticmethod
    def forward(ctx, x, norm_w, eps, w1, w3, w2):
        C = require()
        st = status_word(x.device)
        w13 = fused_bf16((w1, w3))
        b2 = bf16_of(w2)
        x2 = _rows(x)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        nw = norm_w.detach()
        if nw.dtype not in (torch.float32, x2.dtype):
            nw = nw.to(x2.dtype)
        nw = nw.contiguous()
        xn, rstd = C.rmsnorm_fwd(x2, nw, eps)
        m, h = x2.shape[0], w13.shape[0] // 2
        gu = torch.empty((m, 2 * h), dtype=BF16, device=x.device)
        if MLP_FUSE_FWD:
            act = torch.empty((m, h), dtype=BF16, device=x.device)
            C.gemm_swiglu_fwd(xn, w13, gu, act, st)
        else:
            gemm(xn, w13, out=gu)
            act = C.swiglu_fwd(gu[:, :h], gu[:, h:])
        y = torch.empty_like(x)
        gemm(act, b2, out=y.view(m, -1), c=x2, beta=1.0)
        ctx.save_for_backward(x2, nw, rstd, gu, w13, b2)
        ctx.params = (w1, w3, w2)
        ctx.meta = (eps, x.shape, norm_w.dtype)
        ctx.norm_main = getattr(norm_w, "_fm_main_grad", None)
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, dy):
        C = require()
        x2, nw, rstd, gu, w13, b2 = ctx.saved_tensors
        w1, w3, w2 = ctx.params
        eps, x_shape, nw_dtype = ctx.meta
        st = status_word(dy.device)
        dy2 = _rows(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        h = gu.shape[1] // 2
        act = C.swiglu_fwd(gu[:, :h], gu[:, h:])                        # recomputed
        g2 = _weight_grads(ctx.needs_input_grad[5:6], (w2,), dy2, act)
        dgu = torch.empty_like(gu)
        if MLP_FUSE_BWD:
            C.gemm_swiglu_bwd(dy2, b2, gu, dgu, st)
        else:
            dact = gemm(dy2, b2, b_mn=True)
            C.swiglu_bwd(gu[:, :h], gu[:, h:], dact, dgu[:, :h], dgu[:, h:])
        xn, _ = C.rmsnorm_fwd(x2, nw, eps)                              # recomputed
        g13 = _weight_grads(ctx.needs_input_grad[3:5], (w1, w3), dgu, xn)
        dxn = gemm(dgu, w13, b_mn=True)
        dx, dnw = C.rmsnorm_bwd(dxn, x2, nw, rstd, dy2, ctx.needs_input_grad[1], _norm_acc(ctx))
        if dnw is not None and dnw.dtype != nw_dtype:
            dnw = dnw.to(nw_dtype)
        return dx.view(x_shape), dnw, None, g13[0], g13[1], g2[0]


def mlp_block(x, norm_w, eps, w1, w3, w2):
    return _MLPBlock.apply(x, norm_w, eps, w1, w3, w2)


def attention_qkv(qkv, n_q, n_kv, hd, causal=True, rope=None, bt=None):
    """Causal GQA flash attention reading q, k, v as slices of one fused projection output ``[B, T, W]`` (or
    its rows ``[B * T, W]`` with ``bt = (B, T)``); the result is ``[B, T, n_q * hd]``.
    ``rope=(cos, sin)`` rotates the q and k heads of ``qkv`` in place first."""
    if rope is None:
        return _Attention.apply(qkv, n_q, n_kv, hd, causal, None, None, bt)
    if qkv._is_view():          # a view cannot be rotated in place by a node with two outputs: rotate it on its own
        qkv = rope_qkv_(qkv.view(bt[0], bt[1], -1) if qkv.dim() == 2 else qkv, rope[0], rope[1], n_q, n_kv, hd)
        return _Attention.apply(qkv, n_q, n_kv, hd, causal)
    return _Attention.apply(qkv, n_q, n_kv, hd, causal, rope[0], rope[1], bt)[0]


# ------------------------------------------------------------------------------ fused lm_head + cross-entropy
class _LinearCrossEntropy(torch.autograd.Function):
    """``mean CE(h @ W.T, labels)`` without keeping fp32 logits: each chunk of bf16 logits is
    turned into its gradient in place by the loss kernel; the two gradient GEMMs run once in the
    backward over all chunks, scaled by the incoming gradient through a device scalar."""

    @staticmethod
    def forward(ctx, h, weight, labels, chunk, ignore_index):
        C = require()
        w = bf16_of(weight)
        h2 = _rows(h)
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        y = labels.reshape(-1)
        n_tok, V = h2.shape[0], w.shape[0]
        valid = (y != ignore_index).sum().clamp(min=1).to(torch.float32)
        inv_n = valid.reciprocal()
        need_grad = any(ctx.needs_input_grad[:2])
        dlogits = torch.empty((n_tok, V), dtype=BF16, device=h.device)
        row_loss = torch.empty(n_tok, dtype=torch.float32, device=h.device)
        for i in range(0, n_tok, chunk):
            j = min(n_tok, i + chunk)
            gemm(h2[i:j], w, out=dlogits[i:j])
            row_loss[i:j] = C.ce_fwd_bwd(dlogits[i:j], y[i:j], 1.0, inv_n, ignore_index, need_grad)
        total = torch.empty((), dtype=torch.float32, device=h.device)
        C.sum_f32(row_loss, total, 1.0, False)
        ctx.save_for_backward(h2, w, dlogits if need_grad else None)
        ctx.weight = weight
        ctx.h_shape = h.shape
        return total * inv_n

    @staticmethod
    @once_differentiable
    def backward(ctx, g):
        h2, w, dlogits = ctx.saved_tensors
        weight = ctx.weight
        g32 = g.to(torch.float32).reshape(1).contiguous()
        dh = dw = None
        if ctx.needs_input_grad[0]:
            dh = gemm(dlogits, w, b_mn=True, alpha_dev=g32).view(ctx.h_shape)
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "_fm_main_grad", None)
            if main is not None:
                gemm(dlogits, h2, a_mn=True, b_mn=True, out=main, c=main, beta=1.0, alpha_dev=g32, allow_split=True)
            else:
                dw = gemm(dlogits, h2, a_mn=True, b_mn=True, out_dtype=torch.float32, alpha_dev=g32, allow_split=True)
                if dw.dtype != weight.dtype:
                    dw = dw.to(weight.dtype)
        return dh, dw, None, None, None


def linear_cross_entropy(h, weight, labels, chunk=4096, ignore_index=-100):
    return _LinearCrossEntropy.apply(h, weight, labels, int(chunk), int(ignore_index))


# ------------------------------------------------------------------------------ softmax / top-k
class _Softmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y = require().softmax_fwd(x.contiguous())
        ctx.save_for_backward(y)
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        return require().softmax_bwd(y, dy.contiguous())


def softmax_lastdim(x):
    return _Softmax.apply(x)


class _TopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k):
        values, indices = require().topk(x.contiguous(), k)
        ctx.save_for_backward(indices)
        ctx.shape = x.shape
        ctx.mark_non_differentiable(indices)
        return values, indices

    @staticmethod
    @once_differentiable
    def backward(ctx, gv, _gi):
        (indices,) = ctx.saved_tensors
        return gv.new_zeros(ctx.shape).scatter_(-1, indices, gv), None


def topk_lastdim(x, k):
    return _TopK.apply(x, k)
