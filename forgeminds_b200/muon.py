"""Muon: momentum + Newton-Schulz orthogonalised updates for matrices, AdamW for everything else.

One optimizer for a whole model: parameters with ``ndim >= 2`` get the Muon rule (momentum buffer,
optional Nesterov blend, five quintic Newton-Schulz steps, ``sqrt(max(1, rows/cols))`` scaling,
decoupled weight decay), vectors get decoupled AdamW. Behaviour follows the reference's
``forgemind/muon.py:141-275``: gradients and momentum buffers are never mutated by the Nesterov
blend, frozen parameters are skipped, same-shape matrices are orthogonalised as one batch, and with
several ranks each rank orthogonalises every ``world``-th matrix of a bucket and the results are
summed with one all-reduce over ``group`` (pass the replication group when the model is also
tensor/pipeline/expert parallel).

On a B200 the iteration runs on the tcgen05 GEMM with the polynomial folded into the epilogues
(:mod:`forgeminds_b200.ops.newton_schulz`).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

__all__ = ["Muon"]


def _expand_group(spec: dict) -> list:
    """One user group -> concrete groups, split by ``ndim`` unless ``use_muon`` says otherwise."""
    spec = dict(spec)
    params = spec.pop("params")
    params = [params] if isinstance(params, Tensor) else list(params)
    if not params:
        return []
    flag = spec.pop("use_muon", None)
    if flag is None:
        out = []
        matrices = [p for p in params if p.ndim >= 2]
        vectors = [p for p in params if p.ndim < 2]
        if matrices:
            out.append({**spec, "params": matrices, "use_muon": True})
        if vectors:
            out.append({**spec, "params": vectors, "use_muon": False})
        return out
    if flag:
        bad = [tuple(p.shape) for p in params if p.ndim < 2]
        if bad:
            raise ValueError(f"use_muon=True group holds {len(bad)} vector parameter(s), e.g. shape {bad[0]}: "
                             "Muon needs ndim >= 2. Omit use_muon to split automatically or move vectors "
                             "to a use_muon=False group.")
    return [{**spec, "params": params, "use_muon": bool(flag)}]


def _normalise(params, adam_lr: float) -> list:
    items = [params] if isinstance(params, Tensor) else list(params)
    if not items:
        raise ValueError("Muon received an empty parameter iterable")
    if isinstance(items[0], dict):
        groups = [g for spec in items for g in _expand_group(spec)]
        if not groups:
            raise ValueError("Muon received param groups but no parameters")
        return groups
    if not isinstance(items[0], Tensor):
        raise TypeError(f"Muon params must be Tensors or param-group dicts, got {type(items[0]).__name__}")
    groups = _expand_group({"params": items})
    for g in groups:
        if not g["use_muon"]:
            g["lr"] = adam_lr
    return groups


class Muon(torch.optim.Optimizer):
    """``Muon(params, lr=0.02, weight_decay=0, momentum=0.95, nesterov=True, ns_steps=5,
    ns_dtype=torch.bfloat16, betas=(0.9, 0.95), eps=1e-10, adam_lr=None, group=None)``"""

    def __init__(self, params, lr: float = 0.02, weight_decay: float = 0.0, momentum: float = 0.95,
                 nesterov: bool = True, ns_steps: int = 5, ns_dtype: "torch.dtype | None" = torch.bfloat16,
                 betas=(0.9, 0.95), eps: float = 1e-10, adam_lr: "float | None" = None, group=None):
        if ns_steps < 1:
            raise ValueError(f"ns_steps must be >= 1, got {ns_steps}")
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                        ns_steps=ns_steps, ns_dtype=ns_dtype, betas=betas, eps=eps)
        super().__init__(_normalise(params, lr if adam_lr is None else adam_lr), defaults)
        self._dist_group = group

    def add_param_group(self, param_group: dict) -> None:
        for g in _expand_group(param_group):       # validates, and splits by ndim when use_muon is absent
            super().add_param_group(g)

    @torch.no_grad()
    def step(self, closure=None, ctl: "Tensor | None" = None):
        """``ctl`` (optional, 2 floats on the parameters' device: clip coefficient, apply flag) lets a
        training loop enqueue the step before it has read the gradient norm on the host: every gradient
        is multiplied by ``ctl[0]`` and, when ``ctl[1] < 0.5``, parameters, momentum buffers and AdamW
        moments are left exactly as they were (a non-finite gradient cannot leak through a zero
        weight, so the old values are selected, not blended)."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._ctl = None if ctl is None else (ctl[0], ctl[1] > 0.5)
        pg = getattr(self, "_dist_group", None)
        live = dist.is_available() and dist.is_initialized()
        world = dist.get_world_size(pg) if live else 1
        rank = dist.get_rank(pg) if live else 0
        for group in self.param_groups:
            if group["use_muon"]:
                self._muon(group, rank, world, pg)
            else:
                self._adamw(group)
        self._ctl = None
        return loss

    @torch.no_grad()
    def init_state(self) -> None:
        """Create the (zero) state of every trainable parameter that has none yet, so that a state dict
        taken before the first step has the entries a checkpoint loads into."""
        for group in self.param_groups:
            for p in group["params"]:
                if not p.requires_grad or self.state.get(p):
                    continue
                if group["use_muon"]:
                    self.state[p]["momentum_buffer"] = torch.zeros_like(p)
                else:
                    self.state[p].update(exp_avg=torch.zeros_like(p), exp_avg_sq=torch.zeros_like(p), step=0)

    def _gated(self, new: Tensor, old: Tensor) -> Tensor:
        """``new`` when the step applies, ``old`` when the device-side flag says skip."""
        ctl = getattr(self, "_ctl", None)
        return new if ctl is None else torch.where(ctl[1], new, old)

    def _grad_of(self, p: Tensor) -> Tensor:
        g = p.grad if p.grad is not None else torch.zeros_like(p)
        ctl = getattr(self, "_ctl", None)
        return g if ctl is None else g * ctl[0].to(g.dtype)

    # ------------------------------------------------------------------ Muon rule
    def _muon(self, group, rank, world, pg) -> None:
        from .kernels import newton_schulz
        lr, wd, mu = group["lr"], group["weight_decay"], group["momentum"]
        buckets: dict = {}
        for p in group["params"]:
            if not p.requires_grad:
                continue
            if p.ndim < 2:
                raise RuntimeError(f"Muon group received a {p.ndim}-D parameter (shape {tuple(p.shape)}); "
                                   "vectors belong in a use_muon=False group.")
            shape2d = (p.shape[0], p.numel() // p.shape[0])
            buckets.setdefault(shape2d, []).append(p)
        for shape2d, members in buckets.items():
            stack = []
            for p in members:
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p)
                buf = st["momentum_buffer"]
                g = self._grad_of(p)
                buf.copy_(self._gated(buf.lerp(g, 1 - mu), buf))
                direction = g.lerp(buf, mu) if group["nesterov"] else buf
                stack.append(direction.reshape(shape2d).to(torch.float32))
            G = torch.stack(stack)
            ns_dtype = group["ns_dtype"]
            if world > 1:
                ortho = torch.zeros(G.shape, dtype=ns_dtype or G.dtype, device=G.device)
                mine = list(range(rank, G.shape[0], world))
                if mine:
                    ortho[mine] = newton_schulz(G[mine], steps=group["ns_steps"], dtype=ns_dtype).to(ortho.dtype)
                dist.all_reduce(ortho, group=pg)
            else:
                ortho = newton_schulz(G, steps=group["ns_steps"], dtype=ns_dtype)
            gain = max(1.0, shape2d[0] / shape2d[1]) ** 0.5
            for i, p in enumerate(members):
                moved = p * (1 - lr * wd) - ortho[i].reshape(p.shape).to(p.dtype) * (lr * gain)
                p.copy_(self._gated(moved, p))

    # ------------------------------------------------------------------ AdamW rule
    def _adamw(self, group) -> None:
        lr, wd = group["lr"], group["weight_decay"]
        b1, b2 = group["betas"]
        eps = group["eps"]
        for p in group["params"]:
            if not p.requires_grad:
                continue
            g = self._grad_of(p)
            st = self.state[p]
            if "exp_avg" not in st:
                st["exp_avg"] = torch.zeros_like(p)
                st["exp_avg_sq"] = torch.zeros_like(p)
                st["step"] = 0
            st["step"] += 1
            m = st["exp_avg"].lerp(g, 1 - b1)
            v = st["exp_avg_sq"].lerp(g.square(), 1 - b2)
            st["exp_avg"].copy_(self._gated(m, st["exp_avg"]))
            st["exp_avg_sq"].copy_(self._gated(v, st["exp_avg_sq"]))
            m_hat = m / (1 - b1 ** st["step"])
            v_hat = v / (1 - b2 ** st["step"])
            moved = p * (1 - lr * wd) - m_hat / (v_hat.sqrt() + eps) * lr
            p.copy_(self._gated(moved, p))
