"""``Forge``: a small training facade for any ``nn.Module``, plus ``launch`` and ``seed_everything``.

``Forge(model, optimizer, loss_fn=...)`` owns the mechanics of a training step -- device placement
of the batch, autocast (``bf16`` / ``fp16`` with a ``GradScaler``), gradient accumulation with the
loss divided by ``accum``, device-side clipping, non-finite / loss-spike skipping, an optional cosine
schedule, callbacks, checkpoints -- and keeps the budget of one host read per optimizer step. Use it
through ``fit(loader)`` or drive it yourself with ``backward(loss)`` / ``step(batch)``. The interface
and the checkpoint layout (``{"model", "optimizer", "scheduler", "step", "ema_loss", "rng"}`` written
by rank 0 with ``torch.save``, model keys without any wrapper prefix) follow the reference's
``forgemind/forge.py:84-533``.
"""
from __future__ import annotations

import contextlib
import math
import os
import random
import time

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

from .config import OffloadConfig, ParallelConfig
from .data import async_loader, to_device
from .distributed import barrier, cleanup, init_distributed
from .offload import OffloadedAdamW
from .perf import count_host_syncs, warn_once

__all__ = ["Forge", "launch", "ForgeState", "seed_everything"]

_AMP = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


class ForgeState(dict):
    """Metrics of the last optimizer step; keys are also attributes."""

    def __getattr__(self, key):
        try:
            return self[key]
        except KeyError as exc:
            raise AttributeError(key) from exc


def _close(obj) -> None:
    fn = getattr(obj, "close", None)
    if callable(fn):
        fn()


def _unwrap(model):
    return model.module if isinstance(model, nn.parallel.DistributedDataParallel) else model


class Forge:
    def __init__(self, model: nn.Module, optimizer: "torch.optim.Optimizer | None" = None, *, loss_fn=None,
                 device=None, precision: str = "bf16", accum: int = 1, clip: float = 1.0, lr: float = 3e-4,
                 weight_decay: float = 0.1, betas=(0.9, 0.95), eps: float = 1e-8, warmup: int = 0,
                 max_steps: int = 1000, min_lr_ratio: float = 0.1, schedule: "str | None" = None, scheduler=None,
                 compile: bool = False, compile_backend: str = "inductor", compile_mode: str = "default",
                 forward_fn=None, offload: str = "none", fused_ops: bool = False, fused_split_mlp: bool = False,
                 async_batches: bool = True, prefetch_depth: int = 2, seed: int = 1234, log_every: int = 10,
                 skip_nonfinite: bool = True, skip_spike_factor: float = 0.0, callbacks=None, quiet: bool = False):
        if precision not in _AMP:
            raise ValueError(f"precision must be one of {sorted(_AMP)}")
        if accum < 1:
            raise ValueError("accum must be >= 1")
        if offload not in ("none", None, "optimizer"):
            raise ValueError("offload must be 'none' or 'optimizer'")
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.precision, self.amp_dtype = precision, _AMP[precision]
        self.accum, self.clip = int(accum), float(clip)
        self.loss_fn, self.forward_fn = loss_fn, forward_fn
        self.async_batches, self.prefetch_depth = bool(async_batches), max(1, int(prefetch_depth))
        self.quiet, self.log_every, self.seed = quiet, max(1, int(log_every)), seed
        self.max_steps, self.warmup, self.min_lr_ratio = int(max_steps), int(warmup), float(min_lr_ratio)
        self.skip_nonfinite, self.skip_spike_factor = skip_nonfinite, float(skip_spike_factor)
        self.callbacks = list(callbacks or [])
        self.history: list = []
        self.step_count = 0
        self.micro = 0
        self.ema_loss = None
        self._loss_sum = None
        self._last_loss = None
        self._skipped = 0

        torch.manual_seed(seed)
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1
        model = model.to(self.device)
        if fused_ops:
            from .kernels.apply import enable
            enable(model, split=fused_split_mlp)
        if compile:
            if self.device.type == "cpu" and os.environ.get("FORGEMIND_COMPILE_CPU") != "1":
                warn_once("torch.compile skipped on CPU (set FORGEMIND_COMPILE_CPU=1 to force it)", key="forge-compile")
            else:
                model = torch.compile(model, backend=compile_backend, mode=compile_mode)
        self.raw_model = model
        self.model = self._wrap(model)

        if optimizer is None:
            optimizer = torch.optim.AdamW(self.model.parameters(), lr=lr, weight_decay=weight_decay, betas=betas, eps=eps)
        if offload == "optimizer":
            first = optimizer.param_groups[0]
            optimizer = OffloadedAdamW(optimizer.param_groups, lr=first["lr"], betas=first.get("betas", betas),
                                       eps=first.get("eps", eps), cfg=OffloadConfig())
        self.optimizer = optimizer
        self.base_lrs = [g["lr"] for g in optimizer.param_groups]
        self.scheduler = scheduler
        if scheduler is None and schedule == "cosine":
            self.scheduler = torch.optim.lr_scheduler.LambdaLR(optimizer, self._cosine)
        self.scaler = torch.amp.GradScaler("cuda", enabled=True) \
            if precision == "fp16" and self.device.type == "cuda" else None

    # ------------------------------------------------------------------ set-up
    def _wrap(self, model):
        if self.world_size == 1 or isinstance(model, nn.parallel.DistributedDataParallel):
            return model
        ids = [self.device] if self.device.type == "cuda" else None
        return nn.parallel.DistributedDataParallel(model, device_ids=ids)

    def setup(self, model=None, optimizer=None):
        return (self.model if model is None else model, self.optimizer if optimizer is None else optimizer)

    def _cosine(self, step: int) -> float:
        if self.warmup and step < self.warmup:
            return (step + 1) / self.warmup
        t = min(1.0, max(0.0, (step - self.warmup) / max(1, self.max_steps - self.warmup)))
        return self.min_lr_ratio + (1 - self.min_lr_ratio) * 0.5 * (1 + math.cos(math.pi * t))

    def _autocast(self):
        if self.precision == "fp32":
            return contextlib.nullcontext()
        return torch.autocast(device_type=self.device.type, dtype=self.amp_dtype)

    # ------------------------------------------------------------------ step mechanics
    def _run(self, batch):
        if self.forward_fn is not None:
            return self.forward_fn(self.model, batch)
        if isinstance(batch, dict):
            return self.model(**batch)
        if isinstance(batch, (tuple, list)):
            return self.model(*batch)
        return self.model(batch)

    def _loss_of(self, out, batch):
        if self.loss_fn is not None:
            return self.loss_fn(out, batch)
        if torch.is_tensor(out):
            return out
        if isinstance(out, dict) and "loss" in out:
            return out["loss"]
        if isinstance(out, (tuple, list)) and out and torch.is_tensor(out[0]):
            return out[0]
        raise TypeError("cannot infer a loss from the model output; pass loss_fn=")

    def backward(self, loss) -> None:
        """Back-propagate one micro-batch; the loss is divided by ``accum`` here."""
        if loss.dim():
            loss = loss.mean()
        scaled = loss / self.accum
        if self.scaler is not None:
            self.scaler.scale(scaled).backward()
        else:
            scaled.backward()
        self.micro += 1
        self._last_loss = loss.detach()
        part = self._last_loss.float()
        self._loss_sum = part if self._loss_sum is None else self._loss_sum + part

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.optimizer.zero_grad(set_to_none=set_to_none)
        self.micro = 0

    def step(self, batch=None):
        """Run one micro-batch (when given) and update once ``accum`` of them have been seen.
        Returns a :class:`ForgeState` after an update, ``None`` while accumulating."""
        if batch is not None:
            batch = to_device(batch, self.device)
            closing = self.micro + 1 >= self.accum
            ddp = isinstance(self.model, nn.parallel.DistributedDataParallel)
            hold = self.model.no_sync() if (ddp and not closing) else contextlib.nullcontext()
            with hold:
                with self._autocast():
                    out = self._run(batch)
                    loss = self._loss_of(out, batch)
                self.backward(loss)
        if self.micro < self.accum:
            return None
        return self._update()

    @torch.no_grad()
    def _grad_norm(self):
        if self.clip <= 0:
            return None
        own = getattr(self.optimizer, "clip_grad_norm_", None)     # offloaded optimizers hold the gradients
        if callable(own):
            return own(self.clip)
        return torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.clip)

    def _update(self):
        if self.scaler is not None:
            self.scaler.unscale_(self.optimizer)
        gn = self._grad_norm()
        mean_loss = self._loss_sum / max(1, self.micro) if self._loss_sum is not None else self._last_loss.float()
        # the one host read of this optimizer step
        if gn is None:
            (loss_v,), gn_v = torch.stack([mean_loss.float()]).tolist(), float("nan")
        else:
            loss_v, gn_v = torch.stack([mean_loss.float(), gn.detach().float().to(mean_loss.device)]).tolist()
        self._loss_sum = None
        skip = False
        if self.skip_nonfinite or self.skip_spike_factor > 0:
            finite = math.isfinite(loss_v) and (gn is None or math.isfinite(gn_v))
            spike = self.skip_spike_factor > 0 and self.ema_loss is not None and \
                loss_v > self.skip_spike_factor * self.ema_loss
            skip = (self.skip_nonfinite and not finite) or spike or (not finite and self.skip_spike_factor > 0)
        if skip:
            self._skipped += 1
            if self.scaler is not None:
                self.scaler.update()
            self.optimizer.zero_grad(set_to_none=True)
            self.micro = 0
            return ForgeState(step=self.step_count, loss=loss_v, grad_norm=gn_v, skipped=True, lr=self._lr())
        if self.scaler is not None:
            self.scaler.step(self.optimizer)
            self.scaler.update()
        else:
            self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        self.micro = 0
        self.step_count += 1
        if self.scheduler is not None:
            self.scheduler.step()
        state = ForgeState(step=self.step_count, loss=loss_v, grad_norm=gn_v, skipped=False, lr=self._lr())
        if self.skip_spike_factor > 0:
            self.ema_loss = loss_v if self.ema_loss is None else 0.95 * self.ema_loss + 0.05 * loss_v
        self.history.append(dict(state))
        if not self.quiet and self.step_count % self.log_every == 0:
            print(f"step {self.step_count:6d} | loss {loss_v:.4f} | gnorm {gn_v:.3f} | lr {state.lr:.2e}", flush=True)
        for cb in self.callbacks:
            (cb.on_step if hasattr(cb, "on_step") else cb)(self, state)
        return state

    def _lr(self) -> float:
        return self.optimizer.param_groups[0]["lr"]

    # ------------------------------------------------------------------ loops
    def _feed(self, loader):
        return async_loader(loader, self.device, depth=self.prefetch_depth) if self.async_batches else loader

    def fit(self, loader, max_steps=None, epochs: int = 1):
        limit = max_steps or self.max_steps
        done = False
        try:
            for epoch in range(epochs):
                feed = self._feed(loader)            # the prefetching wrapper is one-shot: a new one per epoch
                try:
                    for batch in feed:
                        self.step(batch)
                        if self.step_count >= limit:
                            done = True
                            break
                finally:
                    if feed is not loader:
                        _close(feed)
                for cb in self.callbacks:
                    if hasattr(cb, "on_epoch"):
                        cb.on_epoch(self, epoch)
                if done:
                    break
        finally:
            _close(loader)
        return self.history

    @torch.no_grad()
    def evaluate(self, loader, max_batches: "int | None" = None) -> float:
        feed = self._feed(loader)
        self.model.eval()
        total, n = None, 0
        try:
            for i, batch in enumerate(feed):
                if max_batches is not None and i >= max_batches:
                    break
                batch = to_device(batch, self.device)
                with self._autocast():
                    loss = self._loss_of(self._run(batch), batch)
                total = loss.detach() if total is None else total + loss.detach()
                n += 1
        finally:
            if feed is not loader:
                _close(feed)
            self.model.train()
        return 0.0 if total is None else float(total / n)

    # ------------------------------------------------------------------ checkpoints
    def save(self, path: str) -> None:
        if not dist.is_initialized() or dist.get_rank() == 0:
            os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
            torch.save({"model": _unwrap(self.raw_model).state_dict(),
                        "optimizer": self.optimizer.state_dict(),
                        "scheduler": self.scheduler.state_dict() if self.scheduler else None,
                        "step": self.step_count, "ema_loss": self.ema_loss, "rng": torch.get_rng_state()}, path)
        barrier()

    def load(self, path: str):
        ckpt = torch.load(path, map_location=self.device, weights_only=False)
        _unwrap(self.raw_model).load_state_dict(ckpt["model"])
        self.optimizer.load_state_dict(ckpt["optimizer"])
        if self.scheduler is not None and ckpt.get("scheduler"):
            self.scheduler.load_state_dict(ckpt["scheduler"])
        self.step_count = int(ckpt.get("step", 0))
        self.ema_loss = ckpt.get("ema_loss")
        if "rng" in ckpt:
            torch.set_rng_state(ckpt["rng"].cpu() if torch.is_tensor(ckpt["rng"]) else ckpt["rng"])
        return self

    def count_syncs(self):
        return count_host_syncs()

    def __repr__(self) -> str:
        n = sum(p.numel() for p in self.raw_model.parameters())
        return (f"Forge(model_params={n / 1e6:.2f}M, device={self.device.type}, precision={self.precision}, "
                f"accum={self.accum}, world={self.world_size})")


def seed_everything(seed: int = 1234, workers: bool = False) -> int:
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if workers:
        os.environ.setdefault("PYTHONHASHSEED", str(seed))
    return seed


# ------------------------------------------------------------------------------ launcher
def _init_pure_dp(backend=None):
    if dist.is_initialized():
        return None
    return init_distributed(ParallelConfig(dp_shard=-1), backend=backend)


def _backend() -> str:
    return "nccl" if torch.cuda.is_available() else "gloo"


def _worker(rank: int, world: int, fn, port: int) -> None:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = os.environ["LOCAL_RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    _init_pure_dp(_backend())
    try:
        fn()
    finally:
        cleanup()


def launch(fn=None, nproc: int = 1, port: int = 29517):
    """Decorator (``@launch(nproc=4)``) that runs a module-level function on ``nproc`` processes of
    this host. Under an existing ``torchrun`` (``WORLD_SIZE`` > 1 in the environment) or with
    ``nproc <= 1`` the function simply runs in place after the process group has been initialised."""
    def decorate(f):
        def run(*args, **kwargs):
            if nproc <= 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
                _init_pure_dp(_backend())
                try:
                    return f(*args, **kwargs)
                finally:
                    cleanup()
            if torch.cuda.is_available() and torch.cuda.device_count() < nproc:
                raise RuntimeError(f"nproc={nproc} but only {torch.cuda.device_count()} visible devices")
            import torch.multiprocessing as mp
            return mp.spawn(_worker, args=(nproc, f, port), nprocs=nproc, join=True)
        run.__name__ = getattr(f, "__name__", "launched")
        run.__doc__ = f.__doc__
        return run
    return decorate(fn)() if fn is not None else decorate
