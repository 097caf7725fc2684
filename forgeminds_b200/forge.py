"""``Forge``: two lines turn any ``nn.Module`` into a training loop; plus ``launch`` and ``seed_everything``.

    forge = fm.Forge(model, optimizer, loss_fn=my_loss)
    forge.fit(loader)

What ``Forge`` takes off the user's hands: moving batches to the device, autocast (``bf16``, or ``fp16``
with a gradient scaler), gradient accumulation, clipping on the device, skipping steps whose loss or
gradient norm is not finite (or spikes above a multiple of the running loss), an optional warm-up +
cosine schedule, DDP wrapping when a process group exists, callbacks, and checkpoints. One optimizer
step costs one host read, however many micro-batches it accumulates.

Contract (the reference's ``forgemind/forge.py:84-533``): ``step(batch)`` answers ``None`` while
gradients are still being accumulated and a :class:`ForgeState` once the optimizer has stepped (or the
step was skipped); ``clip=0`` turns clipping off and reports ``grad_norm = nan``; a checkpoint is one
``torch.save`` file with the keys ``model`` (no wrapper prefix), ``optimizer``, ``scheduler``, ``step``,
``ema_loss`` and ``rng``, written by rank 0.
"""
from __future__ import annotations

import contextlib
import math
import os
import random

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

from .config import OffloadConfig, ParallelConfig
from .data import async_loader, to_device
from .distributed import barrier, cleanup, init_distributed
from .perf import count_host_syncs, warn_once

__all__ = ["Forge", "launch", "ForgeState", "seed_everything"]

SPIKE_EMA = 0.95          # weight of the past in the running loss that the spike guard compares against


class ForgeState(dict):
    """What one optimizer step reported (``step, loss, grad_norm, skipped, lr``), readable as attributes."""

    __slots__ = ()

    def __getattr__(self, name):
        if name in self:
            return self[name]
        raise AttributeError(f"ForgeState has no field {name!r}")


class _Amp:
    """Autocast context and, for fp16 on CUDA, the gradient scaler."""

    DTYPES = {"fp32": None, "bf16": torch.bfloat16, "fp16": torch.float16}

    def __init__(self, precision: str, device: torch.device):
        if precision not in self.DTYPES:
            raise ValueError(f"unknown precision {precision!r}; choose from {', '.join(self.DTYPES)}")
        self.name, self.dtype, self.device_type = precision, self.DTYPES[precision], device.type
        self.scaler = torch.amp.GradScaler("cuda") if (precision == "fp16" and device.type == "cuda") else None

    def cast(self):
        if self.dtype is None:
            return contextlib.nullcontext()
        return torch.autocast(self.device_type, dtype=self.dtype)

    def backward(self, loss) -> None:
        (self.scaler.scale(loss) if self.scaler is not None else loss).backward()

    def unscale(self, optimizer) -> None:
        if self.scaler is not None:
            self.scaler.unscale_(optimizer)

    def apply(self, optimizer) -> None:
        if self.scaler is None:
            optimizer.step()
        else:
            self.scaler.step(optimizer)
            self.scaler.update()

    def skipped(self) -> None:
        if self.scaler is not None:          # lets the scaler back off after an overflow
            self.scaler.update()


class _Window:
    """The micro-batches of one optimizer step: how many were seen, and their loss summed on the device."""

    def __init__(self):
        self.seen, self.total, self.last = 0, None, None

    def add(self, loss) -> None:
        self.last = loss.detach()
        piece = self.last.float()
        self.total = piece if self.total is None else self.total + piece
        self.seen += 1

    def mean(self):
        return self.total / self.seen if self.total is not None else self.last.float()

    def clear(self) -> None:
        self.seen, self.total = 0, None


def _is_ddp(m) -> bool:
    return isinstance(m, nn.parallel.DistributedDataParallel)


def _shut(thing) -> None:
    closer = getattr(thing, "close", None)
    if callable(closer):
        closer()


class Forge:
    def __init__(self, model: nn.Module, optimizer: "torch.optim.Optimizer | None" = None, *, loss_fn=None,
                 device=None, precision: str = "bf16", accum: int = 1, clip: float = 1.0, lr: float = 3e-4,
                 weight_decay: float = 0.1, betas=(0.9, 0.95), eps: float = 1e-8, warmup: int = 0,
                 max_steps: int = 1000, min_lr_ratio: float = 0.1, schedule: "str | None" = None, scheduler=None,
                 compile: bool = False, compile_backend: str = "inductor", compile_mode: str = "default",
                 forward_fn=None, offload: str = "none", fused_ops: bool = False, fused_split_mlp: bool = False,
                 async_batches: bool = True, prefetch_depth: int = 2, seed: int = 1234, log_every: int = 10,
                 skip_nonfinite: bool = True, skip_spike_factor: float = 0.0, callbacks=None, quiet: bool = False):
        self.device = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        self.amp = _Amp(precision, self.device)
        if int(accum) < 1:
            raise ValueError(f"accum counts micro-batches per optimizer step and must be at least 1, got {accum}")
        if offload not in (None, "none", "optimizer"):
            raise ValueError(f"offload={offload!r} is not supported here: use 'none' or 'optimizer'")
        self.precision = precision
        self.accum, self.clip = int(accum), float(clip)
        self.loss_fn, self.forward_fn = loss_fn, forward_fn
        self.max_steps, self.warmup, self.min_lr_ratio = int(max_steps), int(warmup), float(min_lr_ratio)
        self.skip_nonfinite, self.skip_spike_factor = bool(skip_nonfinite), float(skip_spike_factor)
        self.async_batches, self.prefetch_depth = bool(async_batches), max(1, int(prefetch_depth))
        self.log_every, self.quiet, self.seed = max(1, int(log_every)), bool(quiet), seed
        self.callbacks = list(callbacks) if callbacks else []
        self.history: list = []
        self.step_count, self.skipped_steps, self.ema_loss = 0, 0, None
        self.window = _Window()

        torch.manual_seed(seed)
        self.world_size = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        self.raw_model = self._prepare(model.to(self.device), fused_ops, fused_split_mlp, compile, compile_backend,
                                       compile_mode)
        self.model = self._data_parallel(self.raw_model)
        self.optimizer = self._optimizer(optimizer, offload, lr, weight_decay, betas, eps)
        self.scheduler = scheduler
        if scheduler is None and schedule == "cosine":
            self.scheduler = torch.optim.lr_scheduler.LambdaLR(self.optimizer, self._lr_factor)

    # ------------------------------------------------------------------ construction
    def _prepare(self, model, fused_ops, fused_split, want_compile, backend, mode):
        if fused_ops:
            from .kernels.apply import enable as patch_in_kernels
            patch_in_kernels(model, split=fused_split)
        if want_compile:
            forced = os.environ.get("FORGEMIND_COMPILE_CPU") == "1"
            if self.device.type == "cpu" and not forced:
                warn_once("Forge(compile=True) is ignored on CPU; FORGEMIND_COMPILE_CPU=1 compiles anyway",
                          key="forge-compile")
            else:
                model = torch.compile(model, backend=backend, mode=mode)
        return model

    def _data_parallel(self, model):
        if self.world_size <= 1 or _is_ddp(model):
            return model
        return nn.parallel.DistributedDataParallel(model, device_ids=[self.device] if self.device.type == "cuda" else None)

    def _optimizer(self, given, offload, lr, weight_decay, betas, eps):
        opt = given
        if opt is None:
            opt = torch.optim.AdamW(self.model.parameters(), lr=lr, weight_decay=weight_decay, betas=betas, eps=eps)
        if offload == "optimizer":
            from .offload import OffloadedAdamW
            head = opt.param_groups[0]
            opt = OffloadedAdamW(opt.param_groups, lr=head["lr"], betas=head.get("betas", betas),
                                 eps=head.get("eps", eps), cfg=OffloadConfig())
        return opt

    def setup(self, model=None, optimizer=None):
        """The (wrapped) model and the optimizer this Forge trains, for code that wants to hold them itself."""
        return (model if model is not None else self.model), (optimizer if optimizer is not None else self.optimizer)

    def _lr_factor(self, step: int) -> float:
        if step < self.warmup:
            return (step + 1) / self.warmup
        span = max(1, self.max_steps - self.warmup)
        frac = min(1.0, max(0.0, (step - self.warmup) / span))
        return self.min_lr_ratio + (1.0 - self.min_lr_ratio) * (1.0 + math.cos(math.pi * frac)) / 2.0

    # ------------------------------------------------------------------ one micro-batch
    def _forward(self, batch):
        if self.forward_fn is not None:
            out = self.forward_fn(self.model, batch)
        elif isinstance(batch, dict):
            out = self.model(**batch)
        elif isinstance(batch, (list, tuple)):
            out = self.model(*batch)
        else:
            out = self.model(batch)
        if self.loss_fn is not None:
            return self.loss_fn(out, batch)
        if torch.is_tensor(out):
            return out
        if isinstance(out, dict) and "loss" in out:
            return out["loss"]
        if isinstance(out, (list, tuple)) and len(out) and torch.is_tensor(out[0]):
            return out[0]
        raise TypeError(f"the model returned {type(out).__name__}, from which no loss can be taken: return a tensor, "
                        "a dict with a 'loss' entry or a tuple whose first element is the loss, or pass loss_fn")

    def backward(self, loss) -> None:
        """Back-propagate one micro-batch's loss, scaled by ``1 / accum`` (and by the fp16 scaler)."""
        if loss.dim() > 0:
            loss = loss.mean()
        self.amp.backward(loss / self.accum)
        self.window.add(loss)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.optimizer.zero_grad(set_to_none=set_to_none)
        self.window.clear()

    def step(self, batch=None):
        """Feed one micro-batch (optional) and, once ``accum`` of them are in, update.

        Returns ``None`` while accumulating and a :class:`ForgeState` after the update."""
        if batch is not None:
            batch = to_device(batch, self.device)
            last_of_window = self.window.seen + 1 >= self.accum
            quiet_ddp = _is_ddp(self.model) and not last_of_window       # no all-reduce for partial sums
            with (self.model.no_sync() if quiet_ddp else contextlib.nullcontext()):
                with self.amp.cast():
                    loss = self._forward(batch)
                self.backward(loss)
        if self.window.seen < self.accum:
            return None
        return self._finish_window()

    # ------------------------------------------------------------------ the optimizer step
    @torch.no_grad()
    def _clipped_norm(self):
        """Total gradient norm as a device tensor (gradients clipped in place), or ``None`` when clipping is off."""
        if self.clip <= 0:
            return None
        own = getattr(self.optimizer, "clip_grad_norm_", None)       # an offloaded optimizer holds the gradients
        if callable(own):
            return own(self.clip)
        return torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.clip)

    def _verdict(self, loss_v: float, norm_v: float) -> bool:
        """True when this step must not be applied."""
        guarded = self.skip_nonfinite or self.skip_spike_factor > 0
        if not guarded:
            return False
        if not (math.isfinite(loss_v) and (math.isnan(norm_v) and self.clip <= 0 or math.isfinite(norm_v))):
            return True
        return self.skip_spike_factor > 0 and self.ema_loss is not None and \
            loss_v > self.skip_spike_factor * self.ema_loss

    def _finish_window(self):
        self.amp.unscale(self.optimizer)
        norm = self._clipped_norm()
        scalars = [self.window.mean()]
        if norm is not None:
            scalars.append(norm.detach().float().to(scalars[0].device))
        numbers = torch.stack(scalars).tolist()            # the only host read of this optimizer step
        loss_v = numbers[0]
        norm_v = numbers[1] if norm is not None else float("nan")
        self.window.clear()
        if self._verdict(loss_v, norm_v):
            self.skipped_steps += 1
            self.amp.skipped()
            self.optimizer.zero_grad(set_to_none=True)
            return ForgeState(step=self.step_count, loss=loss_v, grad_norm=norm_v, skipped=True, lr=self._lr_now())
        self.amp.apply(self.optimizer)
        self.optimizer.zero_grad(set_to_none=True)
        self.step_count += 1
        if self.scheduler is not None:
            self.scheduler.step()
        if self.skip_spike_factor > 0:
            self.ema_loss = loss_v if self.ema_loss is None else SPIKE_EMA * self.ema_loss + (1 - SPIKE_EMA) * loss_v
        state = ForgeState(step=self.step_count, loss=loss_v, grad_norm=norm_v, skipped=False, lr=self._lr_now())
        self.history.append(dict(state))
        if not self.quiet and self.step_count % self.log_every == 0:
            print(f"[forge] step {self.step_count} loss {loss_v:.4f} grad-norm {norm_v:.3f} lr {state.lr:.3g}", flush=True)
        for cb in self.callbacks:
            getattr(cb, "on_step", cb)(self, state)
        return state

    def _lr_now(self) -> float:
        return self.optimizer.param_groups[0]["lr"]

    # ------------------------------------------------------------------ loops
    def _stream(self, loader):
        """The loader itself, or a one-shot prefetching wrapper around it (a fresh one per pass)."""
        if not self.async_batches:
            return loader
        return async_loader(loader, self.device, depth=self.prefetch_depth)

    def fit(self, loader, max_steps=None, epochs: int = 1):
        budget = self.max_steps if not max_steps else max_steps
        try:
            for epoch in range(epochs):
                stream = self._stream(loader)
                try:
                    for batch in stream:
                        self.step(batch)
                        if self.step_count >= budget:
                            break
                finally:
                    if stream is not loader:
                        _shut(stream)
                for cb in self.callbacks:
                    hook = getattr(cb, "on_epoch", None)
                    if hook is not None:
                        hook(self, epoch)
                if self.step_count >= budget:
                    break
        finally:
            _shut(loader)
        return self.history

    @torch.no_grad()
    def evaluate(self, loader, max_batches: "int | None" = None) -> float:
        """Mean loss over ``loader`` (at most ``max_batches`` of it) in eval mode; one host read at the end."""
        stream = self._stream(loader)
        was_training = self.model.training
        self.model.eval()
        acc, count = None, 0
        try:
            for batch in stream:
                if max_batches is not None and count >= max_batches:
                    break
                batch = to_device(batch, self.device)
                with self.amp.cast():
                    loss = self._forward(batch).detach()
                acc = loss if acc is None else acc + loss
                count += 1
        finally:
            if stream is not loader:
                _shut(stream)
            self.model.train(was_training)
        return float(acc / count) if count else 0.0

    # ------------------------------------------------------------------ checkpoints
    def _bare(self):
        return self.raw_model.module if _is_ddp(self.raw_model) else self.raw_model

    def save(self, path: str) -> None:
        writer = not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0
        if writer:
            folder = os.path.dirname(os.path.abspath(path))
            os.makedirs(folder, exist_ok=True)
            blob = {"model": self._bare().state_dict(), "optimizer": self.optimizer.state_dict(),
                    "scheduler": None if self.scheduler is None else self.scheduler.state_dict(),
                    "step": self.step_count, "ema_loss": self.ema_loss, "rng": torch.get_rng_state()}
            torch.save(blob, path)
        barrier()

    def load(self, path: str):
        blob = torch.load(path, map_location=self.device, weights_only=False)
        self._bare().load_state_dict(blob["model"])
        self.optimizer.load_state_dict(blob["optimizer"])
        if self.scheduler is not None and blob.get("scheduler") is not None:
            self.scheduler.load_state_dict(blob["scheduler"])
        self.step_count = int(blob.get("step", 0))
        self.ema_loss = blob.get("ema_loss")
        rng = blob.get("rng")
        if rng is not None:
            torch.set_rng_state(rng.cpu() if torch.is_tensor(rng) else rng)
        return self

    def count_syncs(self):
        """Context manager that counts host<->device synchronisations (see :func:`fm.count_host_syncs`)."""
        return count_host_syncs()

    def __repr__(self) -> str:
        millions = sum(p.numel() for p in self.raw_model.parameters()) / 1e6
        return (f"Forge({type(self._bare()).__name__}, {millions:.2f}M parameters, device={self.device.type}, "
                f"precision={self.precision}, accum={self.accum}, world={self.world_size})")


def seed_everything(seed: int = 1234, workers: bool = False) -> int:
    """Seed Python, NumPy and torch (all CUDA devices). ``workers=True`` also fixes ``PYTHONHASHSEED`` for
    processes started later, unless it is set already."""
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    np.random.seed(seed & 0xFFFFFFFF)
    random.seed(seed)
    if workers and "PYTHONHASHSEED" not in os.environ:
        os.environ["PYTHONHASHSEED"] = str(seed)
    return seed


# ------------------------------------------------------------------------------ launcher
def _join_data_parallel():
    """Bring up the process group as pure data parallelism (every rank a replica), unless one exists."""
    if dist.is_available() and dist.is_initialized():
        return
    init_distributed(ParallelConfig(dp_shard=-1), backend="nccl" if torch.cuda.is_available() else "gloo")


def _child(rank: int, world: int, port: int, fn, args, kwargs) -> None:
    os.environ.update(MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    _join_data_parallel()
    try:
        fn(*args, **kwargs)
    finally:
        cleanup()


def launch(fn=None, nproc: int = 1, port: int = 29517):
    """``@fm.launch(nproc=4)`` runs a module-level function once per process on this host.

    When the script already runs under ``torchrun`` (``WORLD_SIZE > 1``) or ``nproc <= 1``, the function
    is called in this process with the process group initialised; otherwise ``nproc`` children are
    spawned (rendezvous on ``127.0.0.1:port``), each joins the group, calls the function and leaves.
    A failing child fails the call."""
    def wrap(target):
        def launched(*args, **kwargs):
            under_launcher = int(os.environ.get("WORLD_SIZE", "1")) > 1
            if under_launcher or nproc <= 1:
                _join_data_parallel()
                try:
                    return target(*args, **kwargs)
                finally:
                    cleanup()
            if torch.cuda.is_available() and torch.cuda.device_count() < nproc:
                raise RuntimeError(f"launch(nproc={nproc}) needs {nproc} GPUs, this host shows {torch.cuda.device_count()}")
            import torch.multiprocessing as mp
            mp.spawn(_child, args=(nproc, port, target, args, kwargs), nprocs=nproc, join=True)
            return None
        launched.__name__ = getattr(target, "__name__", "launched")
        launched.__qualname__ = getattr(target, "__qualname__", launched.__name__)
        launched.__doc__ = target.__doc__
        launched.__wrapped__ = target
        return launched
    if fn is not None:
        return wrap(fn)()
    return wrap
