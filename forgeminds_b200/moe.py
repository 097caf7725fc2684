"""Mixture of experts: top-k router, SwiGLU experts, expert parallelism.

Module tree and state-dict keys follow the reference's ``forgemind/moe.py:80-287``
(``router.gate.weight [E, d]``, ``experts.w1/w3 [E_local, d, h]``, ``experts.w2 [E_local, h, d]`` in
``x @ w`` layout, ``shared.*``). Routing maths is the reference's: fp32 softmax over the gate logits,
top-k, renormalised weights, Switch load-balance term ``E * sum_e frac_e * mean_tokens(p_e)`` and
z-loss ``mean(logsumexp^2)``.

Three execution paths share those semantics:

* **PyTorch** (CPU, fp32, Gloo): stable sort by expert, per-expert products, ``index_add`` combine;
  expert parallelism through ``all_to_all_single`` with one host read of the split sizes.
* **sm_100a, one GPU**: router softmax/top-k/statistics in one kernel, a device-side slot plan
  (no host read), gather into expert-major rows, grouped tcgen05 GEMMs, weighted combine.
* **sm_100a, expert parallel**: the dispatch writes routed rows straight into the owning rank's
  symmetric buffer and the combine reads them back over NVLink (:mod:`forgeminds_b200.parallel.ep`).

``capacity_factor > 0`` bounds every expert to ``ceil(cf * tokens * top_k / E)`` rows and drops the
overflow (the reference is dropless; 0 keeps that behaviour).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["MoE", "Router", "Experts"]


def _histogram(idx_flat: torch.Tensor, n: int) -> torch.Tensor:
    """Per-expert counts with a static output shape (int64 ``[n]``)."""
    return torch.zeros(n, dtype=torch.int64, device=idx_flat.device).scatter_add_(
        0, idx_flat, torch.ones_like(idx_flat, dtype=torch.int64))


class _AllToAll(torch.autograd.Function):
    """``all_to_all_single`` with uneven row splits whose backward is the reverse exchange."""

    @staticmethod
    def forward(ctx, x, recv_rows, send_rows, group):
        ctx.recv_rows, ctx.send_rows, ctx.group = recv_rows, send_rows, group
        out = x.new_empty((sum(recv_rows),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), recv_rows, send_rows, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        back = g.new_empty((sum(ctx.send_rows),) + tuple(g.shape[1:]))
        dist.all_to_all_single(back, g.contiguous(), ctx.send_rows, ctx.recv_rows, group=ctx.group)
        return back, None, None, None


class Router(nn.Module):
    def __init__(self, dim: int, n_experts: int, top_k: int):
        super().__init__()
        self.gate = nn.Linear(dim, n_experts, bias=False)
        self.n_experts, self.top_k = n_experts, top_k

    def forward(self, x):
        """``x [N, d]`` -> ``(weights [N, k] in x.dtype, idx [N, k], aux, z)``"""
        logits = self.gate(x).float()
        probs = logits.softmax(dim=-1)
        w, idx = probs.topk(self.top_k, dim=-1)
        w = w / w.sum(dim=-1, keepdim=True)
        with torch.no_grad():
            frac = _histogram(idx.reshape(-1), self.n_experts) / idx.numel()
        aux = self.n_experts * (frac * probs.mean(dim=0)).sum()
        z = logits.logsumexp(dim=-1).square().mean()
        return w.to(x.dtype), idx, aux, z


class Experts(nn.Module):
    """SwiGLU experts: stacked ``[E, d, h]`` / ``[E, h, d]`` parameters, or one parameter per expert
    (``ParameterList`` in pinned host memory) when expert offload is on."""

    def __init__(self, n_local: int, dim: int, hidden: int, offload: bool = False, grouped_mm: bool = False):
        super().__init__()
        self.n_local, self.offload = n_local, bool(offload)
        self.dim, self.hidden = dim, hidden
        self.grouped = bool(grouped_mm) and not self.offload
        if self.offload:
            def make(a, b):
                return nn.ParameterList([nn.Parameter(torch.empty(a, b)) for _ in range(n_local)])
        else:
            def make(a, b):
                return nn.Parameter(torch.empty(n_local, a, b))
        self.w1, self.w3, self.w2 = make(dim, hidden), make(dim, hidden), make(hidden, dim)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for group in (self.w1, self.w3, self.w2):
            for p in (group if self.offload else [group]):
                nn.init.normal_(p.data, std=0.02)
                if self.offload and torch.cuda.is_available():
                    p.data = p.data.pin_memory()

    def _weight(self, name: str, e: int, device, dtype):
        w = getattr(self, name)[e]
        if w.device != device:
            w = w.to(device, non_blocking=True)      # streamed on demand; the gradient flows back to the host copy
        return w if w.dtype == dtype else w.to(dtype)

    def forward(self, x, counts=None, offsets=None):
        """``x`` holds the routed rows grouped by local expert; ``counts`` (list or tensor) or
        cumulative ``offsets`` give the group sizes."""
        if counts is None:
            if offsets is None:
                counts = [x.shape[0]]
            else:
                ends = offsets.to(torch.int64)
                counts = torch.diff(ends, prepend=ends.new_zeros(1)).tolist()
        elif torch.is_tensor(counts):
            counts = counts.tolist()
        sizes = [int(c) for c in counts]
        outs = []
        start = 0
        for e, n_rows in enumerate(sizes):
            if n_rows:
                rows = x[start:start + n_rows]
                a = self._weight("w1", e, x.device, x.dtype)
                b = self._weight("w3", e, x.device, x.dtype)
                o = self._weight("w2", e, x.device, x.dtype)
                outs.append((F.silu(rows @ a) * (rows @ b)) @ o)
            start += n_rows
        if not outs:
            return x.new_zeros((0,) + tuple(x.shape[1:]))
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=0)


class MoE(nn.Module):
    def __init__(self, dim, hidden, n_experts, top_k, n_shared=0, ep_size=1, ep_group=None, ep_rank=0,
                 offload_experts=False, grouped_mm=False, aux_coef=1e-2, z_coef=1e-3, capacity_factor=0.0):
        super().__init__()
        assert n_experts % ep_size == 0, "n_experts must be divisible by ep_size"
        self.dim, self.hidden = dim, hidden
        self.n_experts, self.top_k = n_experts, top_k
        self.ep_size, self.ep_group, self.ep_rank = ep_size, ep_group, ep_rank
        self.n_local = n_experts // ep_size
        self.router = Router(dim, n_experts, top_k)
        self.experts = Experts(self.n_local, dim, hidden, offload=offload_experts, grouped_mm=grouped_mm)
        self.shared = None
        if n_shared:
            from .models.gpt import SwiGLU
            self.shared = SwiGLU(dim, hidden * n_shared)
        self.aux_coef, self.z_coef = aux_coef, z_coef
        self.capacity_factor = float(capacity_factor or 0.0)
        self.last_aux: Optional[torch.Tensor] = None
        self.ep_engine = None            # set by parallel.ep.attach() for the fused NVLink path

    @property
    def compile_friendly(self) -> bool:
        return self.ep_size == 1 and self.experts.grouped

    def probe_grouped(self, device, dtype) -> bool:
        """Decide once, before the first step, whether the device path (no host read) can run."""
        e = self.experts
        if not e.grouped:
            return False
        ok = torch.device(device).type == "cuda" and dtype == torch.bfloat16
        if ok:
            from . import ops
            ok = ops.available()
        e.grouped = bool(ok)
        return e.grouped

    def capacity(self, n_tokens: int) -> int:
        if self.capacity_factor <= 0:
            return 0
        return int(math.ceil(self.capacity_factor * n_tokens * self.top_k / self.n_experts))

    # ------------------------------------------------------------------ forward
    def forward(self, x):
        shape = x.shape
        flat = x.reshape(-1, self.dim)
        if self._use_native(flat):
            from .ops.moe import moe_forward_native
            out = moe_forward_native(self, flat)
            return out.reshape(shape)
        w, idx, aux, z = self.router(flat)
        self.last_aux = self.aux_coef * aux + self.z_coef * z
        out = self._dispatch_torch(flat, w, idx)
        if self.shared is not None:
            out = out + self.shared(flat)
        return out.reshape(shape)

    def _use_native(self, flat) -> bool:
        if not (flat.is_cuda and flat.dtype == torch.bfloat16) or self.experts.offload:
            return False
        if self.ep_size > 1 and self.ep_engine is None:
            return False
        from . import ops
        return ops.available() and self.dim % 64 == 0 and self.hidden % 64 == 0 and self.n_experts <= 256 \
            and self.top_k <= 8

    def _dispatch_torch(self, flat, w, idx):
        n_tok = flat.shape[0]
        choice = idx.reshape(-1)
        gate = w.reshape(-1)
        cap = self.capacity(n_tok)
        if cap:
            # position of every routed entry inside its expert (stable), entries past the capacity drop out
            one_hot = F.one_hot(choice, self.n_experts)
            pos = (one_hot.cumsum(dim=0) - 1).gather(1, choice[:, None]).squeeze(1)
            keep = pos < cap
            gate = gate * keep.to(gate.dtype)
        order = torch.sort(choice, stable=True).indices
        token = order // self.top_k
        rows = flat[token]
        counts = _histogram(choice, self.n_experts)
        if self.ep_size == 1:
            ys = self.experts(rows, counts=counts)
        else:
            ys = self._exchange(rows, counts)
        ys = ys * gate[order].unsqueeze(-1)
        return torch.zeros_like(flat).index_add_(0, token, ys.to(flat.dtype))

    def _exchange(self, rows, counts):
        """Expert-parallel exchange over ``torch.distributed`` (Gloo/NCCL): counts all-to-all, one
        host read for every split size, token all-to-all, experts, and the way back."""
        E_l, ep = self.n_local, self.ep_size
        mine = counts.view(ep, E_l)
        theirs = torch.empty_like(mine)
        dist.all_to_all_single(theirs.view(-1), mine.contiguous().view(-1), group=self.ep_group)
        host = torch.cat([mine.sum(dim=1), theirs.reshape(-1)]).tolist()          # the single host read
        send = [int(v) for v in host[:ep]]
        table = [[int(v) for v in host[ep + r * E_l: ep + (r + 1) * E_l]] for r in range(ep)]   # [src][expert]
        recv = [sum(r) for r in table]
        got = _AllToAll.apply(rows, recv, send, self.ep_group)                    # ordered [src][expert]
        # regroup by expert so that each expert sees one contiguous block
        pieces, cursor = {}, 0
        for r in range(ep):
            for e in range(E_l):
                pieces[(r, e)] = got[cursor: cursor + table[r][e]]
                cursor += table[r][e]
        by_expert = [torch.cat([pieces[(r, e)] for r in range(ep)], dim=0) for e in range(E_l)]
        per_expert = [sum(table[r][e] for r in range(ep)) for e in range(E_l)]
        outs = []
        for e in range(E_l):
            if per_expert[e]:
                sizes = [per_expert[e] if i == e else 0 for i in range(E_l)]
                outs.append(self.experts(by_expert[e], counts=sizes))
            else:
                outs.append(by_expert[e])
        # back to [src][expert] order, then home
        back = {}
        for e in range(E_l):
            parts = outs[e].split([table[r][e] for r in range(ep)], dim=0)
            for r in range(ep):
                back[(r, e)] = parts[r]
        ordered = torch.cat([back[(r, e)] for r in range(ep) for e in range(E_l)], dim=0)
        return _AllToAll.apply(ordered, send, recv, self.ep_group)
