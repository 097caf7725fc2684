"""Tensor parallelism with sequence-parallel activations, fused with its collectives.

Inside the stack of blocks the residual stream is split by rows (tokens) over the ``tp`` ranks:
rank r holds rows ``[r * Ms, (r + 1) * Ms)`` of the ``[M, d]`` activations. Every linear layer of a
block is then one kernel that does its collective while it computes (``csrc/gemm_sm100.cu``, PEER
instantiations):

* column-parallel ``wq|wk|wv`` and ``w1|w3``: **all-gather -> GEMM**. Each rank publishes its
  normalised rows in its slice of a symmetric ``[M, d]`` buffer. Two extra warps of every CTA of the
  GEMM pull the other ranks' slices into the local buffer -- every row crosses NVLink once -- and count
  arrived rows per 128-row block; the TMA producer reads local memory only, multiplies this rank's own
  rows first and waits (bounded) for a block's count before it touches it.
* row-parallel ``wo`` and ``w2``: **GEMM -> reduce-scatter**. The epilogue stores each 128-row tile of
  the bf16 partial product into the staging buffer of the rank that owns those rows (slice = source
  rank), remote rows first; after a flag barrier the owner sums the slices (fp32, fixed order) together
  with the residual.

The backward uses the same two kernels: the input gradient of a column-parallel layer is a
GEMM -> reduce-scatter, its weight gradient an all-gather -> GEMM with the gathered operand on the
reduction side; for a row-parallel layer the roles swap (and its second product reuses the rows the
first one gathered).

Buffer protocol (one :class:`TPState` per group). Two gather buffers ``[M, d]`` (activations,
gradients) and one staging buffer ``[W, Ms, d]``. A publish is always separated from the previous
product that read the same slice by a full flag barrier (every reduce-scatter ends with one), and a
peer can only reach its next reduce-scatter into a rank's staging buffer after waiting for that rank's
next publish, which comes after the rank has summed the buffer.

Blocks whose projections are int8 / fp8 layers run the same layout with the 8-bit tensor-core products of
``csrc/gemm8_sm100.cu`` between NCCL all-gather / reduce-scatter calls (:func:`quant_gather_linear`,
:func:`quant_linear_scatter`): the gather warps and the scattered-output epilogue exist in the bf16 kernel only.

The reference expresses the same layout with DTensor ``ColwiseParallel`` / ``RowwiseParallel`` and
NCCL all-reduces (``forgemind/parallel/native.py:21-49``); that path remains the fallback
(:func:`usable` false: CPU, Gloo, ``fused_comm=False``, shapes that do not tile).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch.autograd.function import once_differentiable

from .. import ops

BF16 = torch.bfloat16


def usable(ctx) -> bool:
    pc = ctx.pc
    return bool(getattr(pc, "fused_comm", True)) and ctx.device.type == "cuda" and ops.available() \
        and 1 < pc.tp <= 8 and pc.ep == 1


class TPState:
    """Symmetric buffers, flag slots and epochs of one tensor-parallel group."""

    def __init__(self, group, device, timeout_ms: float = 10000.0):
        from .symm import SymmGroup
        self.sg = SymmGroup(group, device, timeout_ms=timeout_ms)
        self.group = group
        self.rank, self.world = self.sg.rank, self.sg.world
        self.slot_act, self.slot_grad, self.slot_bar = (self.sg.reserve_slots(1) for _ in range(3))
        self._bufs: dict = {}
        self.quant_calls = 0          # 8-bit column-parallel products issued so far (tests read it)

    def buffers(self, rows: int, width: int):
        """(gather buffer for activations, gather buffer for gradients, staging) for row shards ``[rows, width]``:
        the gather buffers hold ``[world * rows, width]``, the staging buffer ``[world, rows, width]``."""
        key = (rows, width)
        if key not in self._bufs:
            sg, w = self.sg, self.world
            self._bufs[key] = (sg.alloc(w * rows * width, BF16), sg.alloc(w * rows * width, BF16),
                               sg.alloc(w * rows * width, BF16),
                               torch.zeros(max(1, w * rows // 128), dtype=torch.int32, device=sg.device))
        return self._bufs[key]

    def publish(self, buf, slot: int, shard: torch.Tensor) -> int:
        """Copy ``shard`` into this rank's slice of the gather buffer and tell the peers; returns the epoch."""
        rows = shard.shape[0]
        buf.local.view(self.world * rows, -1)[self.rank * rows:(self.rank + 1) * rows].copy_(shard)
        epoch = self.sg.next_epoch(slot)
        ops.require().comm_signal(self.sg.flags.ptrs, slot, epoch, self.rank, self.sg.status)
        return epoch

    def gemm(self, a, b, out, a_mn=False, b_mn=False, accumulate=False, gather=0, gather_buf=None, ready=None,
             d_buf=None, wait=(-1, 0)):
        sg = self.sg
        ops.require().gemm_peer(a, b, out, a_mn, b_mn, 1.0, accumulate, self.rank, self.world, gather,
                                gather_buf.ptrs if gather else [], ready if gather else None,
                                d_buf.ptrs if d_buf is not None else [], sg.flags.local, wait[0], wait[1],
                                sg.timeout_ms, sg.status)
        return out

    def barrier(self):
        self.sg.barrier(self.slot_bar)

    def reduce(self, staging, rows: int, width: int, residual=None) -> torch.Tensor:
        """Sum of the slices that the ranks stored into this rank's staging buffer (+ residual)."""
        out = torch.empty((rows, width), dtype=BF16, device=self.sg.device)
        ops.require().comm_sum_partials(staging.local, residual, out, self.world)
        return out


def _plain(t, what: str):
    """The kernels take raw device pointers: a DTensor / sharded parameter must never reach them."""
    if hasattr(t, "to_local"):
        raise TypeError(f"fused tensor parallelism got a DTensor for {what}; it needs the full local tensor "
                        "(was the block called directly instead of through its data-parallel wrapper?)")
    return t


def _main_grad_or_new(param, shape, device):
    main = getattr(param, "_fm_main_grad", None)
    if main is not None:
        return main, True
    return torch.empty(shape, dtype=torch.float32, device=device), False


class _GatherLinear(torch.autograd.Function):
    """``all_gather_rows(x_shard) @ cat(W_local...).T`` -> ``[M, sum N_local]`` (column-parallel layers that
    share their input: q|k|v, gate|up). The weights stay separate parameters; when a flat parameter store
    laid their bf16 copies and gradient buffers out back to back the product reads and writes them in
    place, otherwise the concatenation is cached and the gradient is split."""

    @staticmethod
    def forward(ctx, x_shard, tp: TPState, *weights):
        from ..ops.functional import fused_bf16
        for wt in weights:
            _plain(wt, "a column-parallel weight")
        w = fused_bf16(weights)
        ms, k = x_shard.shape
        act, _, _, ready = tp.buffers(ms, k)
        epoch = tp.publish(act, tp.slot_act, x_shard)
        m = ms * tp.world
        y = torch.empty((m, w.shape[0]), dtype=BF16, device=x_shard.device)
        tp.gemm(act.local.view(m, k), w, y, gather=1, gather_buf=act, ready=ready, wait=(tp.slot_act, epoch))
        ctx.save_for_backward(x_shard, w)
        ctx.tp, ctx.weights = tp, weights
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, dy):
        from ..ops.functional import fused_main_grad
        x_shard, w = ctx.saved_tensors
        tp, weights = ctx.tp, ctx.weights
        ms, k = x_shard.shape
        m = ms * tp.world
        act, _, staging, ready = tp.buffers(ms, k)
        dy = dy.contiguous()
        grads = [None] * len(weights)
        if any(ctx.needs_input_grad[2:]):
            # dW[N_l, K] = dy[M, N_l].T @ gather(x)[M, K]: the gathered operand is on the reduction side
            epoch = tp.publish(act, tp.slot_act, x_shard)
            main = fused_main_grad(weights)
            out = main if main is not None else torch.empty(w.shape, dtype=torch.float32, device=dy.device)
            tp.gemm(dy, act.local.view(m, k), out, a_mn=True, b_mn=True, accumulate=main is not None, gather=2,
                    gather_buf=act, ready=ready, wait=(tp.slot_act, epoch))
            if main is None:
                lo = 0
                for i, wt in enumerate(weights):
                    piece = out[lo:lo + wt.shape[0]]
                    lo += wt.shape[0]
                    own = getattr(wt, "_fm_main_grad", None)
                    if own is not None:
                        own.add_(piece)
                    elif ctx.needs_input_grad[2 + i]:
                        grads[i] = piece.to(wt.dtype)
        dx = None
        if ctx.needs_input_grad[0]:
            # dx_shard = reduce_scatter_rows(dy @ W_local)
            tp.gemm(dy, w, staging.local.view(m, k), b_mn=True, d_buf=staging)
            tp.barrier()
            dx = tp.reduce(staging, ms, k)
        return (dx, None, *grads)


class _LinearScatter(torch.autograd.Function):
    """``reduce_scatter_rows(h @ W_local.T) (+ residual_shard)`` -> ``[Ms, N]`` (row-parallel layer)."""

    @staticmethod
    def forward(ctx, h, weight, residual, tp: TPState):
        from ..ops.functional import bf16_of
        w = bf16_of(_plain(weight, "a row-parallel weight"))
        m, n = h.shape[0], w.shape[0]
        ms = m // tp.world
        _, _, staging, _ = tp.buffers(ms, n)
        h = h.contiguous()
        tp.gemm(h, w, staging.local.view(m, n), d_buf=staging)
        tp.barrier()
        out = tp.reduce(staging, ms, n, residual.contiguous() if residual is not None else None)
        ctx.save_for_backward(h, w)
        ctx.tp, ctx.weight, ctx.has_res = tp, weight, residual is not None
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, dout):
        h, w = ctx.saved_tensors
        tp, weight = ctx.tp, ctx.weight
        ms, n = dout.shape
        m = ms * tp.world
        _, grad, _, ready = tp.buffers(ms, n)
        dout = dout.contiguous()
        epoch = tp.publish(grad, tp.slot_grad, dout)
        full = grad.local.view(m, n)
        dh = dw = None
        gathered = False
        if ctx.needs_input_grad[0]:
            # dh[M, K_l] = gather(dout)[M, N] @ W_local[N, K_l]
            dh = torch.empty_like(h)
            tp.gemm(full, w, dh, b_mn=True, gather=1, gather_buf=grad, ready=ready, wait=(tp.slot_grad, epoch))
            gathered = True
        if ctx.needs_input_grad[1]:
            # dW[N, K_l] = gather(dout)[M, N].T @ h[M, K_l]; the rows are already here after the product above
            out, is_main = _main_grad_or_new(weight, w.shape, dout.device)
            if gathered:
                tp.gemm(full, h, out, a_mn=True, b_mn=True, accumulate=is_main)
            else:
                tp.gemm(full, h, out, a_mn=True, b_mn=True, accumulate=is_main, gather=1, gather_buf=grad, ready=ready,
                        wait=(tp.slot_grad, epoch))
            dw = None if is_main else out.to(weight.dtype)
        return dh, dw, (dout if ctx.has_res else None), None


def gather_linear(x_shard, weights, tp: TPState):
    """``weights``: one weight or a tuple of weights whose outputs are concatenated."""
    if isinstance(weights, torch.Tensor):
        weights = (weights,)
    return _GatherLinear.apply(x_shard, tp, *weights)


def linear_scatter(h, weight, residual, tp: TPState):
    return _LinearScatter.apply(h, weight, residual, tp)


class _TakeShard(torch.autograd.Function):
    """Rows ``[r * Ms, (r + 1) * Ms)`` of a replicated ``[M, d]`` tensor; the gradient of the other rows
    is produced by the ranks that own them."""

    @staticmethod
    def forward(ctx, x, rank, world):
        ms = x.shape[0] // world
        ctx.meta = (rank, world, x.shape)
        return x[rank * ms:(rank + 1) * ms].contiguous()

    @staticmethod
    def backward(ctx, dx):
        rank, world, shape = ctx.meta
        full = dx.new_zeros(shape)
        ms = shape[0] // world
        full[rank * ms:(rank + 1) * ms] = dx
        return full, None, None


class _GatherRows(torch.autograd.Function):
    """All-gather of row shards (NCCL); the consumer runs replicated, so the backward keeps this rank's rows."""

    @staticmethod
    def forward(ctx, x_shard, group, rank, world):
        out = x_shard.new_empty((x_shard.shape[0] * world,) + tuple(x_shard.shape[1:]))
        dist.all_gather_into_tensor(out, x_shard.contiguous(), group=group)
        ctx.meta = (rank, world)
        return out

    @staticmethod
    def backward(ctx, dout):
        rank, world = ctx.meta
        ms = dout.shape[0] // world
        return dout[rank * ms:(rank + 1) * ms].contiguous(), None, None, None


class _AllGatherRows(torch.autograd.Function):
    """All-gather of row shards whose consumer is column-parallel (every rank multiplies ALL rows by its own
    weight slice): the input gradient is the sum of the ranks' partial gradients, reduce-scattered back."""

    @staticmethod
    def forward(ctx, x_shard, group, world):
        out = x_shard.new_empty((x_shard.shape[0] * world,) + tuple(x_shard.shape[1:]))
        dist.all_gather_into_tensor(out, x_shard.contiguous(), group=group)
        ctx.group, ctx.world = group, world
        return out

    @staticmethod
    def backward(ctx, dout):
        dx = dout.new_empty((dout.shape[0] // ctx.world,) + tuple(dout.shape[1:]))
        dist.reduce_scatter_tensor(dx, dout.contiguous(), group=ctx.group)
        return dx, None, None


class _ReduceScatterRows(torch.autograd.Function):
    """Sum of the ranks' partial outputs of a row-parallel layer, each rank keeping its rows."""

    @staticmethod
    def forward(ctx, y_partial, group, world):
        out = y_partial.new_empty((y_partial.shape[0] // world,) + tuple(y_partial.shape[1:]))
        dist.reduce_scatter_tensor(out, y_partial.contiguous(), group=group)
        ctx.group, ctx.world = group, world
        return out

    @staticmethod
    def backward(ctx, dout):
        full = dout.new_empty((dout.shape[0] * ctx.world,) + tuple(dout.shape[1:]))
        dist.all_gather_into_tensor(full, dout.contiguous(), group=ctx.group)
        return full, None, None


def quant_gather_linear(x_shard, linears, tp: TPState):
    """Column-parallel projection(s) of int8 / fp8 layers: the row shards are all-gathered (NCCL) and multiplied
    by this rank's weight slices as ONE product on the 8-bit tensor-core kernel. The bf16 kernels above fuse the
    gather into the product; the 8-bit kernel has no gather warps, so here the collective is a call of its own."""
    from ..ops.quant import qlinear_multi
    tp.quant_calls += 1
    x_full = _AllGatherRows.apply(x_shard, tp.group, tp.world)
    head = linears[0]
    return qlinear_multi(x_full, tuple(m.weight for m in linears), head.mode, head.block)


def quant_linear_scatter(h, linear, residual, tp: TPState):
    """Row-parallel int8 / fp8 projection: 8-bit product of this rank's columns, reduce-scatter of the bf16
    partial outputs (NCCL), residual added to the rows this rank keeps."""
    return _ReduceScatterRows.apply(linear(h), tp.group, tp.world) + residual


# ---------------------------------------------------------------------------------------------- model surgery
def _shard_rows(linear, lo, hi):
    w = linear.weight.data[lo:hi].clone()
    linear.weight = torch.nn.Parameter(w)
    linear.out_features = hi - lo
    linear.weight._tp_shard_dim = 0


def _shard_cols(linear, lo, hi):
    w = linear.weight.data[:, lo:hi].clone()
    linear.weight = torch.nn.Parameter(w)
    linear.in_features = hi - lo
    linear.weight._tp_shard_dim = 1


def shard_model(model, ctx, plan=None):
    """Give every block its slice of the attention heads and of the MLP width and switch the model
    to the sequence-parallel forward. Parameters that stay replicated but see only this rank's rows
    (block norms, embedding) are marked: their gradients are summed over the group before clipping
    (:func:`sync_partial_grads`)."""
    cfg = model.cfg
    tp, rank = ctx.pc.tp, ctx.tp_rank
    hd = cfg.dim // cfg.n_heads
    state = TPState(ctx.tp_group, ctx.device, timeout_ms=float(getattr(ctx.pc, "comm_timeout_ms", 10000)))
    for blk in model.layers.values():
        at, ff = blk.attn, blk.ffn
        if not hasattr(at, "wq") or not hasattr(ff, "w1"):
            raise RuntimeError("fused tensor parallelism covers attention + SwiGLU blocks")
        nq, nkv = cfg.n_heads // tp, cfg.n_kv_heads // tp
        _shard_rows(at.wq, rank * nq * hd, (rank + 1) * nq * hd)
        _shard_rows(at.wk, rank * nkv * hd, (rank + 1) * nkv * hd)
        _shard_rows(at.wv, rank * nkv * hd, (rank + 1) * nkv * hd)
        _shard_cols(at.wo, rank * nq * hd, (rank + 1) * nq * hd)
        hidden = ff.w1.weight.shape[0]
        if hidden % tp:
            raise ValueError(f"MLP width {hidden} does not divide over tp={tp}")
        hl = hidden // tp
        _shard_rows(ff.w1, rank * hl, (rank + 1) * hl)
        _shard_rows(ff.w3, rank * hl, (rank + 1) * hl)
        _shard_cols(ff.w2, rank * hl, (rank + 1) * hl)
        blk.attn_norm.weight._tp_partial = True
        blk.ffn_norm.weight._tp_partial = True
        blk._fm_tp = state
    if getattr(model, "tok_emb", None) is not None:           # absent on all but the first pipeline stage
        model.tok_emb.weight._tp_partial = True
    model._fm_tp = state
    return model


def sync_partial_grads(model, state: TPState) -> None:
    """Sum, over the tensor-parallel group, the gradients of replicated parameters that were computed
    from this rank's rows only."""
    grads = [p.grad for p in model.parameters() if getattr(p, "_tp_partial", False) and p.grad is not None]
    for g in grads:
        dist.all_reduce(g, group=state.group)


def block_forward(blk, x_shard, state: TPState):
    """One transformer block on a row shard ``[Ms, d]`` of the residual stream."""
    from ..models.gpt import rope_tables
    from ..ops import functional as Fn
    from ..models.gpt import _is_quantised
    at, ff = blk.attn, blk.ffn
    hd = at.hd
    nq, nkv = at.wq.weight.shape[0] // hd, at.wk.weight.shape[0] // hd
    q_attn, q_ffn = _is_quantised(at.wq), _is_quantised(ff.w1)      # int8 / fp8 layers: 8-bit products, NCCL collectives
    xn = Fn.rms_norm(x_shard, blk.attn_norm.weight, blk.attn_norm.eps)
    if q_attn:
        qkv = quant_gather_linear(xn, (at.wq, at.wk, at.wv), state)
    else:
        qkv = gather_linear(xn, (at.wq.weight, at.wk.weight, at.wv.weight), state)     # [M, (nq + 2 nkv) * hd]
    B, T = blk._fm_bt
    cos, sin = rope_tables(T, hd, at.theta, qkv.device, torch.float32)
    o = Fn.attention_qkv(qkv, nq, nkv, hd, True,                # rows in, [B, T, nq * hd] out
                         rope=(cos.reshape(T, hd // 2), sin.reshape(T, hd // 2)), bt=(B, T))
    o = o.reshape(B * T, nq * hd)
    h = quant_linear_scatter(o, at.wo, x_shard, state) if _is_quantised(at.wo) else \
        linear_scatter(o, at.wo.weight, x_shard, state)
    hn = Fn.rms_norm(h, blk.ffn_norm.weight, blk.ffn_norm.eps)
    if q_ffn:
        gu = quant_gather_linear(hn, (ff.w1, ff.w3), state)
    else:
        gu = gather_linear(hn, (ff.w1.weight, ff.w3.weight), state)               # [M, 2 * hidden_local]
    act = Fn.swiglu_split(gu)
    return quant_linear_scatter(act, ff.w2, h, state) if _is_quantised(ff.w2) else \
        linear_scatter(act, ff.w2.weight, h, state)


def stack_forward(model, x):
    """Blocks of ``model`` on ``x [B, T, d]`` (replicated): shard rows, run the blocks, gather."""
    state = model._fm_tp
    B, T, d = x.shape
    if (B * T) % (128 * state.world):
        raise ValueError(f"fused tensor parallelism needs B*T ({B * T}) to be a multiple of {128 * state.world}")
    xs = _TakeShard.apply(x.reshape(B * T, d).to(BF16), state.rank, state.world)
    for blk in model.layers.values():
        blk._fm_bt = (B, T)
        xs = blk(xs)          # through __call__: data-parallel wrappers (FSDP2 / DDP hooks) must see the call
    full = _GatherRows.apply(xs, state.group, state.rank, state.world)
    return full.view(B, T, d)
