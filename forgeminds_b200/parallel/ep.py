"""Expert parallelism over peer memory (``csrc/moe_ep.cu``): no ``all_to_all`` and no host read.

Rank r owns experts ``[r * E_local, (r + 1) * E_local)``. Per MoE layer and direction the ranks
exchange only flags; the payload moves inside the permutation kernels:

forward
  1. route locally; publish token rows, expert ids (and keep the weights) in symmetric buffers;
  2. every rank renumbers ALL ranks' expert ids for its own experts and plans slots on the device;
  3. slot rows are pulled from the tokens' ranks (dispatch), grouped SwiGLU GEMMs run locally;
  4. every token pulls its k outputs from the owners' buffers through the owners' slot tables (combine).
backward
  the owners pull ``dout`` rows and routing weights, run the expert backward, and the tokens' ranks
  pull ``dx`` rows back the same way; ``d(loss)/d(routing weight)`` is pushed to the token's rank.

Buffers are shared by all layers of a model; a flag barrier at the end of each layer call keeps a
fast rank from overwriting what a slow one still reads. Slot buffers are sized for the worst case
(every token of every rank choosing this rank's experts); the GEMMs skip row tiles without live rows.

The reference exchanges split sizes with ``all_to_all_single``, reads them on the host, and moves
the rows with two more all-to-alls around a sort and ``index_add_`` (``forgemind/moe.py:62-79,227-287``).
"""
from __future__ import annotations

import torch
from torch.autograd.function import once_differentiable

from .. import ops
from ..ops.moe import ALIGN          # rows: expert regions start on multiples of it (256-row tiles on CTA pairs)

BF16 = torch.bfloat16


def bounded_rows(slots: int, entries: int, world: int, e_local: int, factor: float) -> int:
    """Rows of a rank's dispatch buffers: the worst case ``slots`` (every routed row of every rank lands here),
    or ``factor`` times the rank's average share plus the padding of its expert regions when that is less."""
    if factor <= 0:
        return slots
    want = int(factor * entries / world) + e_local * ALIGN
    return min(slots, (want + ALIGN - 1) // ALIGN * ALIGN)


def clamp_plan(region, limit, rows: int):
    """Cut a slot plan down to ``rows`` buffer rows (device tensors in, device tensors out, no host read):
    expert regions ``[start, used, padded]`` end at ``rows``, and so does the first row past the live ones.
    Returns ``(region, limit, overflowed)`` with ``overflowed`` a device bool."""
    over = limit[0] > rows
    limit = limit.clone()
    limit[0] = torch.clamp(limit[0], max=rows)
    r = region.view(-1, 3).clone()
    end_pad = torch.clamp(r[:, 0] + r[:, 2], max=rows)
    end_use = torch.clamp(r[:, 0] + r[:, 1], max=rows)
    r[:, 0] = torch.clamp(r[:, 0], max=rows)
    r[:, 2] = end_pad - r[:, 0]
    r[:, 1] = end_use - r[:, 0]
    return r.view(region.shape), limit, over


class EPEngine:
    def __init__(self, group, device, timeout_ms: float = 10000.0, slot_factor: float = 0.0):
        from .symm import SymmGroup
        self.slot_factor = float(slot_factor)
        self.sg = SymmGroup(group, device, timeout_ms=timeout_ms)
        self.rank, self.world = self.sg.rank, self.sg.world
        sg = self.sg
        self.s_pub, self.s_ys, self.s_gpub, self.s_dxs, self.s_done = (sg.reserve_slots(1) for _ in range(5))
        self._key = None

    def _buffers(self, n: int, k: int, d: int, slots: int):
        key = (n, k, d, slots)
        if self._key != key:
            sg = self.sg
            self.x_sym = sg.alloc(n * d, BF16)                   # token rows (forward) / dout rows (backward)
            self.idx_sym = sg.alloc(n * k, torch.int32)
            self.w_sym = sg.alloc(n * k, torch.float32)          # routing weights (backward)
            self.drw_sym = sg.alloc(n * k, torch.float32)        # gradient of the routing weights, pushed by the owners
            self.slot_sym = sg.alloc(self.world * n * k, torch.int32)
            self.rows_sym = sg.alloc(slots * d, BF16)            # expert outputs (forward) / expert input grads (backward)
            self._key = key
        return self

    def signal(self, slot: int) -> int:
        epoch = self.sg.next_epoch(slot)
        ops.require().comm_signal(self.sg.flags.ptrs, slot, epoch, self.rank, self.sg.status)
        return epoch

    # ------------------------------------------------------------------ layer entry point
    def forward(self, moe, x):
        """``x [N, d]`` bf16 -> ``[N, d]``; sets ``moe.last_aux``."""
        from ..ops.functional import linear
        from ..ops.moe import _Route
        gate = moe.router.gate.weight
        if gate.shape[0] % 8 == 0:
            logits = linear(x, gate)
        else:
            logits = torch.nn.functional.linear(x, gate.to(x.dtype))
        route_w, idx, aux, _counts = _Route.apply(logits, moe.top_k, moe.aux_coef, moe.z_coef)
        moe.last_aux = aux
        ex = moe.experts
        out = _EPExperts.apply(x, route_w, idx, ex.w1, ex.w3, ex.w2, self, moe.n_experts, moe.capacity(x.shape[0]))
        if moe.shared is not None:
            from ..ops.functional import linear_multi, swiglu_linear
            gu = linear_multi(x, (moe.shared.w1.weight, moe.shared.w3.weight))
            out = swiglu_linear(gu, moe.shared.w2.weight, out)
        return out


class _EPExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, route_w, idx, w1, w3, w2, eng: EPEngine, n_experts: int, capacity: int):
        from ..ops.functional import bf16_of
        C = ops.require()
        sg, W, rank = eng.sg, eng.world, eng.rank
        st = sg.status
        n, d = x.shape
        k = idx.shape[1]
        e_local = w1.shape[0]
        assert e_local * W == n_experts, "experts must divide evenly over the expert-parallel group"
        h = w1.shape[2]
        entries = W * n * k
        if capacity > 0:
            cap = (capacity * W + ALIGN - 1) // ALIGN * ALIGN    # capacity counts tokens of all ranks
            slots = (e_local + 1) * cap
        else:
            cap = 0
            slots = (entries + ALIGN - 1) // ALIGN * ALIGN + (e_local + 1) * ALIGN
        plan_slots = slots
        if not cap:        # dropless: the row buffers may be smaller than the plan's worst case
            slots = bounded_rows(plan_slots, entries, W, e_local, eng.slot_factor)
        eng._buffers(n, k, d, slots)
        # 1. publish
        eng.x_sym.local.view(n, d).copy_(x)
        eng.idx_sym.local.view(n, k).copy_(idx)
        e_pub = eng.signal(eng.s_pub)
        # 2. plan over the entries of all ranks (the last "expert" collects what other ranks own)
        all_idx = torch.empty((W * n, k), dtype=torch.int32, device=x.device)
        C.ep_collect_idx(eng.idx_sym.ptrs, all_idx, n * k, rank, e_local, sg.flags.local, eng.s_pub, e_pub,
                         sg.timeout_ms, st)
        slot_of, token_of, region, _meta = C.moe_plan(all_idx, e_local + 1, ALIGN, cap, 1 if cap else 0, plan_slots)
        if slots < plan_slots:
            # bounded buffers: rows past them are cut from the plan (one small kernel, in place; `clamp_plan` is its
            # PyTorch statement), and a layer that needed them leaves a code in the status word, which the step
            # reads with its loss (the host is not asked here)
            C.ep_clamp_plan(region, slots, st, ops.ERR_EP_OVERFLOW)
        limit = region[e_local]                                  # [start of the foreign region, ...]: live rows end here
        own = region[:e_local]
        slot_of = torch.where(slot_of >= limit[0], torch.full_like(slot_of, -1), slot_of)   # foreign entries have no slot here
        tile_group = C.moe_tile_groups(own, slots // 128)
        entry_of = torch.full((slots + 1,), -1, dtype=torch.int32, device=x.device)
        entry_of.scatter_(0, torch.where(slot_of >= 0, slot_of, torch.full_like(slot_of, slots)).long(),
                          torch.arange(entries, dtype=torch.int32, device=x.device))
        entry_of[slots] = -1
        eng.slot_sym.local.copy_(slot_of)
        # 3. dispatch + experts
        # Dropless plans have no dead row tile inside an expert's region and nothing below touches rows past
        # `limit`, so the buffers need no clearing. With a capacity an unused tile inside a region would feed
        # stale values into the expert weight gradients: those (bounded) buffers are cleared.
        alloc = torch.zeros if cap else torch.empty
        xs = alloc((slots, d), dtype=BF16, device=x.device)
        C.ep_gather(eng.x_sym.ptrs, token_of, limit, xs, n, sg.flags.local, eng.s_pub, e_pub, sg.timeout_ms, st)
        b1, b3, b2 = bf16_of(w1), bf16_of(w3), bf16_of(w2)
        gu = alloc((slots, 2 * h), dtype=BF16, device=x.device)
        C.gemm_grouped_rows(xs, b1, gu[:, :h], tile_group, True, False, st, True)
        C.gemm_grouped_rows(xs, b3, gu[:, h:], tile_group, True, False, st, True)
        act = C.swiglu_fwd(gu[:, :h], gu[:, h:], limit)
        ys = eng.rows_sym.local.view(slots, d)
        if cap:
            ys.zero_()
        C.gemm_grouped_rows(act, b2, ys, tile_group, True, False, st, True)
        e_ys = eng.signal(eng.s_ys)
        # 4. combine: every token pulls from the owners
        rw = route_w.detach().to(torch.float32).contiguous()
        out = torch.empty((n, d), dtype=BF16, device=x.device)
        C.ep_combine(eng.rows_sym.ptrs, eng.slot_sym.ptrs, idx, rw, out, e_local, rank, sg.flags.local, eng.s_ys,
                     e_ys, sg.timeout_ms, st)
        ys_keep = ys.clone()
        sg.barrier(eng.s_done)
        ctx.save_for_backward(xs, gu, ys_keep, rw, idx, slot_of, entry_of, region, tile_group, b1, b3, b2)
        ctx.params = (w1, w3, w2)
        ctx.eng = eng
        ctx.dims = (n, d, h, k, e_local, slots, route_w.dtype, bool(cap))
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, dout):
        C = ops.require()
        xs, gu, ys, rw, idx, slot_of, entry_of, region, tile_group, b1, b3, b2 = ctx.saved_tensors
        w1, w3, w2 = ctx.params
        eng = ctx.eng
        sg, W, rank = eng.sg, eng.world, eng.rank
        st = sg.status
        n, d, h, k, e_local, slots, rw_dtype, clear = ctx.dims
        alloc = torch.zeros if clear else torch.empty
        limit, own = region[e_local], region[:e_local]
        # publish what the owners need: output gradient rows, routing weights, this layer's slot table
        eng.x_sym.local.view(n, d).copy_(dout)
        eng.w_sym.local.copy_(rw.view(-1))
        eng.slot_sym.local.copy_(slot_of)
        eng.drw_sym.local.zero_()            # entries dropped by a capacity limit get no push: their gradient is zero
        e_g = eng.signal(eng.s_gpub)
        dys = alloc((slots, d), dtype=BF16, device=dout.device)
        C.ep_combine_bwd(eng.x_sym.ptrs, eng.w_sym.ptrs, eng.drw_sym.ptrs, ys, entry_of, limit, dys, n * k, k,
                         sg.flags.local, eng.s_gpub, e_g, sg.timeout_ms, st)
        act = C.swiglu_fwd(gu[:, :h], gu[:, h:], limit)                       # recomputed
        grads = {}

        def wgrad(name, param, a, b):
            main = getattr(param, "_fm_main_grad", None)
            if main is not None:
                C.gemm_grouped_wgrad(a, b, main, own, True, st)
                grads[name] = None
            else:
                g = torch.empty(param.shape, dtype=torch.float32, device=dout.device)
                C.gemm_grouped_wgrad(a, b, g, own, False, st)
                grads[name] = g if g.dtype == param.dtype else g.to(param.dtype)

        wgrad("w2", w2, act, dys)
        dact = alloc((slots, h), dtype=BF16, device=dout.device)
        C.gemm_grouped_rows(dys, b2, dact, tile_group, False, False, st, True)
        dgu = alloc(gu.shape, dtype=BF16, device=dout.device)
        C.swiglu_bwd(gu[:, :h], gu[:, h:], dact, dgu[:, :h], dgu[:, h:], limit)
        wgrad("w1", w1, xs, dgu[:, :h])
        wgrad("w3", w3, xs, dgu[:, h:])
        dxs = eng.rows_sym.local.view(slots, d)
        if clear:
            dxs.zero_()
        C.gemm_grouped_rows(dgu[:, :h], b1, dxs, tile_group, False, False, st, True)
        C.gemm_grouped_rows(dgu[:, h:], b3, dxs, tile_group, False, True, st, True)
        e_dx = eng.signal(eng.s_dxs)
        dx = torch.empty((n, d), dtype=BF16, device=dout.device)
        C.ep_combine(eng.rows_sym.ptrs, eng.slot_sym.ptrs, idx, None, dx, e_local, rank, sg.flags.local, eng.s_dxs,
                     e_dx, sg.timeout_ms, st)
        drw = eng.drw_sym.local.clone().view(n, k).to(rw_dtype)
        sg.barrier(eng.s_done)
        return dx, drw, None, grads["w1"], grads["w3"], grads["w2"], None, None, None


def attach(model, ctx) -> EPEngine:
    """Give every MoE layer of ``model`` the peer-memory expert-parallel engine of ``ctx.ep_group``."""
    eng = EPEngine(ctx.ep_group, ctx.device, timeout_ms=float(getattr(ctx.pc, "comm_timeout_ms", 10000)),
                   slot_factor=float(getattr(ctx.pc, "ep_slot_factor", 0.0)))
    hits = 0
    for m in model.modules():
        if hasattr(m, "ep_engine") and getattr(m, "ep_size", 1) > 1:
            m.ep_engine = eng
            hits += 1
    if not hits:
        raise RuntimeError("ep.attach: the model has no expert-parallel MoE layer")
    model._fm_ep = eng
    return eng
