"""Offload of optimizer state, gradients and saved activations to pinned host memory.

``OffloadedAdamW`` keeps fp32 master weights and AdamW moments on the host; gradients leave the
GPU on a side stream as soon as autograd has produced them (post-accumulate hooks) and the host
update of one chunk of parameters overlaps the device->host copies of the next. ``ActivationOffload``
spills large saved-for-backward tensors of a block to pooled pinned buffers. Behaviour and knobs
follow the reference's ``forgemind/offload.py:40-322``; all copies are ``cudaMemcpyAsync`` on
dedicated streams (``Tensor.copy_(non_blocking=True)`` from/to pinned memory).
"""
from __future__ import annotations

import time

import torch
import torch.nn as nn

from .config import OffloadConfig
from .perf import _PinnedPool

__all__ = ["OffloadedAdamW", "ActivationOffload", "apply_activation_offload"]


def _memory_pressure() -> float:
    if not torch.cuda.is_available():
        return 0.0
    free, total = torch.cuda.mem_get_info()
    return 1.0 - free / total


class OffloadedAdamW:
    """AdamW with master weights and moments in (pinned) host memory.

    Not for sharded (DTensor) parameters. Call :meth:`collect` after a backward when hooks are off
    (``overlap=False``); :meth:`step` applies the update and copies the new weights back.
    """

    def __init__(self, param_groups, lr, betas=(0.9, 0.95), eps=1e-8, cfg: OffloadConfig = None, overlap=True):
        self.cfg = cfg or OffloadConfig()
        self.params = [p for g in param_groups for p in g["params"]]
        assert self.params, "OffloadedAdamW got no parameters (all frozen?)"
        assert not any(hasattr(p, "to_local") for p in self.params), \
            "OffloadedAdamW does not support DTensor/FSDP parameters"
        self.cuda = any(p.is_cuda for p in self.params)
        self.stream = torch.cuda.Stream() if self.cuda else None
        self.n_chunks = max(1, int(getattr(self.cfg, "pipeline_chunks", 4)))
        self._chunk = {p: i % self.n_chunks for i, p in enumerate(self.params)}
        self._chunk_events = [torch.cuda.Event() for _ in range(self.n_chunks)] if self.cuda else None
        self.stats = {"d2h_bytes": 0, "d2h_ops": 0, "h2d_bytes": 0, "h2d_ops": 0, "syncs": 0,
                      "host_update_ms": 0.0, "stream_ms": 0.0}
        self.master, self.cgrad = {}, {}
        host_groups = []
        for g in param_groups:
            hosted = []
            for p in g["params"]:
                m = p.detach().to("cpu", torch.float32, copy=True)
                acc = torch.zeros_like(m)
                if self.cuda:
                    m, acc = m.pin_memory(), acc.pin_memory()
                m.grad = acc
                self.master[p], self.cgrad[p] = m, acc
                hosted.append(m)
            host_groups.append({**{k: v for k, v in g.items() if k != "params"}, "params": hosted})
        self.opt = torch.optim.AdamW(host_groups, lr=lr, betas=betas, eps=eps)
        self.param_groups = self.opt.param_groups
        self._accs = [self.cgrad[p] for p in self.params]
        self._staging: dict = {}
        self._has_value: set = set()
        self._in_flight: list = []          # (param, staging buffer or None)
        self._pressure = 0.0
        self.hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in self.params] if overlap else []

    # ------------------------------------------------------------------ gradient streaming
    def begin_step(self) -> None:
        if self.cfg.smart and self.cfg.gpu_watermark > 0:
            self._pressure = _memory_pressure()

    def _wants(self, p) -> bool:
        if not self.cfg.smart:
            return True
        if p.numel() < self.cfg.min_numel:
            return False
        return self.cfg.gpu_watermark <= 0 or self._pressure >= self.cfg.gpu_watermark

    def _on_grad(self, p) -> None:
        if p.grad is not None and self._wants(p):
            self._move(p)

    def _move(self, p) -> None:
        g = p.grad
        if g is None:
            return
        p.grad = None
        acc = self.cgrad[p]
        if not (self.cuda and g.is_cuda):
            acc.add_(g)
            self._has_value.add(p)
            return
        self.stream.wait_stream(torch.cuda.current_stream())
        if p in self._has_value:
            buf = self._staging.get(p)
            if buf is None or buf.dtype != g.dtype:
                buf = self._staging[p] = torch.empty(p.shape, dtype=g.dtype, device="cpu", pin_memory=True)
            target = buf
        else:
            target, buf = acc, None         # the accumulator is zero: a copy into it is the accumulate
            self._has_value.add(p)
        with torch.cuda.stream(self.stream):
            target.copy_(g, non_blocking=True)
        g.record_stream(self.stream)
        self._in_flight.append((p, buf))
        self._chunk_events[self._chunk[p]].record(self.stream)
        self.stats["d2h_ops"] += 1
        self.stats["d2h_bytes"] += g.numel() * g.element_size()

    def collect(self) -> None:
        """Move every gradient still on the device to the host accumulators and wait for them."""
        for p in self.params:
            if p.grad is not None:
                self._move(p)
        self.flush()

    def flush(self) -> None:
        if not self._in_flight:
            return
        if self.cuda:
            self.stats["syncs"] += 1
            self.stream.synchronize()
            for p, buf in self._in_flight:
                if buf is not None:
                    self.cgrad[p].add_(buf)
        self._in_flight.clear()

    # ------------------------------------------------------------------ optimizer interface
    @torch.no_grad()
    def clip_grad_norm_(self, max_norm):
        self.collect()
        norm = torch.linalg.vector_norm(torch.stack(torch._foreach_norm(self._accs)))
        if max_norm and max_norm > 0:
            torch._foreach_mul_(self._accs, torch.clamp(max_norm / (norm + 1e-6), max=1.0))
        return norm

    @torch.no_grad()
    def step(self) -> None:
        t0 = time.perf_counter()
        if self.n_chunks <= 1:
            self.collect()
        else:
            for p in self.params:
                if p.grad is not None:
                    self._move(p)
            by_chunk = [[] for _ in range(self.n_chunks)]
            for p, buf in self._in_flight:
                by_chunk[self._chunk[p]].append((p, buf))
            for k, items in enumerate(by_chunk):
                if not items:
                    continue
                if self._chunk_events is not None:
                    self._chunk_events[k].synchronize()      # only this chunk's copies
                    self.stats["syncs"] += 1
                for p, buf in items:
                    if buf is not None:
                        self.cgrad[p].add_(buf)
            self._in_flight.clear()
        self.stats["stream_ms"] += (time.perf_counter() - t0) * 1e3
        t1 = time.perf_counter()
        self.opt.step()
        self.stats["host_update_ms"] += (time.perf_counter() - t1) * 1e3
        for p in self.params:
            p.data.copy_(self.master[p], non_blocking=self.cuda)      # stream-ordered; no host wait
            if self.cuda:
                self.stats["h2d_ops"] += 1
                self.stats["h2d_bytes"] += p.numel() * p.element_size()
        self._clear()

    def _clear(self) -> None:
        torch._foreach_zero_(self._accs)
        self._has_value.clear()

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.flush()
        for p in self.params:
            p.grad = None
        self._clear()

    def state_dict(self) -> dict:
        return {"opt": self.opt.state_dict(), "master": [self.master[p] for p in self.params]}

    def load_state_dict(self, sd: dict) -> None:
        self.opt.load_state_dict(sd["opt"])
        for p, m in zip(self.params, sd["master"]):
            self.master[p].copy_(m)
            p.data.copy_(self.master[p])
        self._clear()

    def report(self) -> dict:
        out = dict(self.stats)
        out["d2h_MB"] = round(out["d2h_bytes"] / 2 ** 20, 2)
        out["h2d_MB"] = round(out["h2d_bytes"] / 2 ** 20, 2)
        out["chunks"] = self.n_chunks
        out["params"] = len(self.params)
        out["grad_bytes_MB"] = round(sum(p.numel() * p.element_size() for p in self.params) / 2 ** 20, 2)
        return out

    def __repr__(self) -> str:
        n = sum(p.numel() for p in self.params)
        return f"OffloadedAdamW(params={len(self.params)}, {n / 1e6:.1f}M, device={'cuda' if self.cuda else 'cpu'})"


class ActivationOffload(torch.autograd.graph.saved_tensors_hooks):
    """Saved-tensor hooks that park CUDA activations of at least ``min_bytes`` in pinned host
    buffers (parameters and leaf tensors stay on the device)."""

    def __init__(self, min_bytes: int = 1 << 20, pool: "_PinnedPool | None" = None):
        self.pool = pool
        pinned = torch.cuda.is_available()

        def pack(t):
            small = t.numel() * t.element_size() < min_bytes
            if not t.is_cuda or small or isinstance(t, nn.Parameter) or (t.requires_grad and t.is_leaf):
                return None, t
            host = pool.get(t.shape, t.dtype) if pool is not None else \
                torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=pinned)
            host.copy_(t, non_blocking=True)
            return t.device, host

        def unpack(packed):
            device, payload = packed
            if device is None:
                return payload
            back = payload.to(device, non_blocking=True)
            if pool is not None:
                pool.put(payload)              # reusable once this stream-ordered copy has been issued
            return back

        super().__init__(pack, unpack)


def apply_activation_offload(model, cfg: OffloadConfig):
    """Wrap the first ``act_layers`` fraction of ``model.layers`` so their saved activations spill."""
    blocks = list(model.layers.values())
    n = max(1, int(len(blocks) * cfg.act_layers)) if blocks else 0
    pool = _PinnedPool(pin=torch.cuda.is_available()) if cfg.act_pool else None
    for blk in blocks[:n]:
        hook = ActivationOffload(cfg.act_min_bytes, pool)
        inner = blk.forward

        def wrapped(*a, _inner=inner, _hook=hook, **k):
            with _hook:
                return _inner(*a, **k)
        blk.forward = wrapped
    return model
