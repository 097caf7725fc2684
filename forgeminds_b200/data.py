"""Datasets, a resumable data-parallel sampler and the asynchronous batch pipeline.

The pipeline keeps batch construction and the host->device copy off the critical path: a
producer thread pulls from the loader, issues the copy from pinned memory on a dedicated CUDA
stream and attaches an event; the consumer makes its compute stream wait on that event on the
device, so the host never blocks. Public surface and semantics follow the reference's
``forgemind/data.py:58-640`` (``SyntheticLM``, ``TokenFile``, ``ResumableSampler``,
``BatchStream``, ``async_loader``, ``build_loader``, ``to_device``).
"""
from __future__ import annotations

import contextlib
import queue
import threading
import time

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, Sampler

from .perf import warn_once

__all__ = ["SyntheticLM", "TokenFile", "ResumableSampler", "BatchStream", "build_loader",
           "async_loader", "to_device", "RandomTokens"]


# ------------------------------------------------------------------------------ datasets
class SyntheticLM(Dataset):
    """Learnable toy corpus: each sample is a concatenation of 8-token motifs drawn from a bank
    of 16, so a small model drives the loss down within a few dozen steps."""

    def __init__(self, vocab: int, seq: int, n: int = 4096, seed: int = 0):
        gen = torch.Generator().manual_seed(seed)
        self.motifs = torch.randint(0, vocab, (16, 8), generator=gen)
        self.pick = torch.randint(0, 16, (n, seq // 8 + 2), generator=gen)
        self.seq = seq

    def __len__(self):
        return self.pick.shape[0]

    def __getitem__(self, i):
        row = self.motifs[self.pick[i]].reshape(-1)[: self.seq + 1]
        return {"input_ids": row[:-1], "labels": row[1:]}


class RandomTokens(Dataset):
    """Uniform random tokens with next-token labels (the shape used by the benchmarks)."""

    def __init__(self, vocab: int, seq: int, n: int = 1024, seed: int = 0):
        gen = torch.Generator().manual_seed(seed)
        self.tokens = torch.randint(0, vocab, (n, seq + 1), generator=gen)

    def __len__(self):
        return self.tokens.shape[0]

    def __getitem__(self, i):
        row = self.tokens[i]
        return {"input_ids": row[:-1], "labels": row[1:]}


class TokenFile(Dataset):
    """Flat binary token file (uint16/uint32) read through ``np.memmap`` in windows of ``seq``."""

    def __init__(self, path, seq: int, dtype="uint16"):
        self.path, self.seq = path, seq
        self.dtype = np.dtype(dtype)
        self.data = np.memmap(path, dtype=self.dtype, mode="r")
        self.n = max(0, (len(self.data) - 1) // seq)

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        lo = i * self.seq
        window = torch.from_numpy(np.asarray(self.data[lo: lo + self.seq + 1], dtype=np.int64))
        return {"input_ids": window[:-1], "labels": window[1:]}

    def close(self):
        if getattr(self, "data", None) is not None and len(self.data):
            self.data = np.empty(0, dtype=self.dtype)

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


# ------------------------------------------------------------------------------ sampler
class ResumableSampler(Sampler):
    """Shards sample indices by *data-parallel* rank (tp/pp ranks of one replica read the same
    data), reshuffles per epoch from ``seed + epoch`` and can skip the first ``skip`` indices of
    the next iteration to resume mid-epoch."""

    def __init__(self, n: int, dp_rank: int, dp_world: int, seed: int = 0, shuffle: bool = True):
        self.n, self.r, self.w = n, dp_rank, dp_world
        self.seed, self.shuffle = seed, shuffle
        self.epoch = 0
        self.skip = 0
        self.per_rank = n // dp_world

    def set_epoch(self, epoch: int) -> None:
        self.epoch = int(epoch)

    def __iter__(self):
        if self.shuffle:
            order = torch.randperm(self.n, generator=torch.Generator().manual_seed(self.seed + self.epoch)).tolist()
        else:
            order = list(range(self.n))
        usable = self.n - self.n % self.w
        mine = order[:usable][self.r::self.w]
        start, self.skip = self.skip, 0
        return iter(mine[start:])

    def __len__(self):
        return max(0, self.per_rank - self.skip)


# ------------------------------------------------------------------------------ helpers
def to_device(obj, device, non_blocking: bool = False):
    """Move every tensor inside a nested dict/list/tuple (named tuples kept) to ``device``."""
    if torch.is_tensor(obj):
        return obj if obj.device == torch.device(device) else obj.to(device, non_blocking=non_blocking)
    if isinstance(obj, dict):
        return {k: to_device(v, device, non_blocking) for k, v in obj.items()}
    if isinstance(obj, tuple) and hasattr(obj, "_fields"):
        return type(obj)(*(to_device(v, device, non_blocking) for v in obj))
    if isinstance(obj, tuple):
        return tuple(to_device(v, device, non_blocking) for v in obj)
    if isinstance(obj, list):
        return [to_device(v, device, non_blocking) for v in obj]
    return obj


def _leaves(obj):
    if torch.is_tensor(obj):
        yield obj
    elif isinstance(obj, dict):
        for v in obj.values():
            yield from _leaves(v)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            yield from _leaves(v)


def _finalize_iterator(it) -> None:
    """Stop the worker pool of a persistent DataLoader iterator, if it has one."""
    stop = getattr(it, "_shutdown_workers", None)
    if callable(stop):
        with contextlib.suppress(Exception):
            stop()


def _length(loader):
    try:
        return int(len(loader))
    except (TypeError, AttributeError):
        return None


class _Staged:
    __slots__ = ("payload", "event", "epoch", "index", "epoch_len")

    def __init__(self, payload, event, epoch=0, index=0, epoch_len=None):
        self.payload, self.event = payload, event
        self.epoch, self.index, self.epoch_len = epoch, index, epoch_len


class _Failure:
    __slots__ = ("exc",)

    def __init__(self, exc):
        self.exc = exc


_DONE = object()


class _Copier:
    """Issues host->device copies on a side stream and hands back (device payload, event)."""

    def __init__(self, device, enabled: bool = True):
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device) if (enabled and self.device.type == "cuda") else None

    def stage(self, obj):
        if self.stream is None:
            return to_device(obj, self.device, non_blocking=True), None
        with torch.cuda.stream(self.stream):
            moved = to_device(obj, self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return moved, ev

    @staticmethod
    def join(payload, event):
        """Order the consumer's stream after the copy, on the device."""
        if event is not None:
            cur = torch.cuda.current_stream()
            cur.wait_event(event)
            for t in _leaves(payload):
                t.record_stream(cur)
        return payload


def _bind(device) -> None:
    dev = torch.device(device)
    if dev.type == "cuda":
        with contextlib.suppress(Exception):
            torch.cuda.set_device(dev)


class _Mailbox:
    """Bounded FIFO whose ``put`` gives up as soon as ``stop`` is set."""

    def __init__(self, depth: int):
        self.q: queue.Queue = queue.Queue(maxsize=depth)
        self.stop = threading.Event()

    def put(self, item) -> bool:
        while not self.stop.is_set():
            try:
                self.q.put(item, timeout=0.1)
                return True
            except queue.Full:
                pass
        return False

    def get(self):
        return self.q.get()

    def drain(self):
        with contextlib.suppress(queue.Empty):
            while True:
                self.q.get_nowait()


# ------------------------------------------------------------------------------ BatchStream
class BatchStream:
    """Endless stream of ``(input_ids, labels)`` already on the device.

    ``prefetch``  copy on a side stream (CUDA) ahead of use.
    ``threaded``  run the loader on a producer thread. ``None`` picks it when prefetching and
                  either the device is CUDA or the loader has no workers.
    ``depth``     batches in flight.

    ``epoch`` / ``batches`` describe the position *after* the batch most recently handed out and
    are exact even while the producer runs ahead; :meth:`resume` restarts at a given position.
    """

    def __init__(self, loader, sampler, device, prefetch: bool = True, depth: int = 2,
                 threaded: "bool | None" = None):
        self.loader, self.sampler, self.device = loader, sampler, device
        self.prefetch = bool(prefetch)
        self.depth = max(1, int(depth))
        self._copier = _Copier(device, enabled=self.prefetch)
        self.stream = self._copier.stream
        if threaded is None:
            workers = int(getattr(loader, "num_workers", 0) or 0)
            threaded = self.prefetch and (torch.device(device).type == "cuda" or workers == 0)
            if threaded:
                warn_once("batch prefetch thread enabled: dataset/collate code shares the global torch "
                          "RNG with training; pass threaded=False for bit-exact reproducibility",
                          key="batchstream-rng")
        self.threaded = bool(threaded) and self.prefetch
        self.epoch = 0
        self.batches = 0
        self._from = (0, 0)
        self._epoch_len = _length(loader)
        if self._epoch_len == 0:
            raise self._empty()
        self.stats = {"batches": 0, "wait_ms": 0.0, "stalled": 0, "max_wait_ms": 0.0,
                      "produce_ms": 0.0, "threaded": self.threaded, "depth": self.depth}
        self._box = _Mailbox(self.depth)
        self._thread = None
        self._it = None
        self._ahead = None           # serial mode: the batch staged for the next call
        self._newest = None
        self._closed = False
        self._begin()

    # ---- producer side
    def _open_epoch(self, epoch: int) -> None:
        if hasattr(self.sampler, "set_epoch"):
            self.sampler.set_epoch(epoch)
        self._it = iter(self.loader)

    def _stage(self, batch, epoch, index) -> _Staged:
        t0 = time.perf_counter()
        payload, ev = self._copier.stage((batch["input_ids"], batch["labels"]))
        self.stats["produce_ms"] += (time.perf_counter() - t0) * 1e3
        return _Staged(payload, ev, epoch, index, self._epoch_len)

    def _produce(self) -> None:
        _bind(self.device)
        epoch, index = self._from
        box = self._box
        try:
            while not box.stop.is_set():
                try:
                    batch = next(self._it)
                except StopIteration:
                    # the epoch ended here: record its true length on the last item handed over
                    self._epoch_len = index or None
                    if self._newest is not None and self._newest.epoch == epoch:
                        self._newest.epoch_len = index
                    epoch, index = epoch + 1, 0
                    self._open_epoch(epoch)
                    try:
                        batch = next(self._it)
                    except StopIteration:
                        box.put(_DONE)
                        return
                if box.stop.is_set():
                    return
                item = self._stage(batch, epoch, index)
                if not box.put(item):
                    return
                self._newest = item
                index += 1
                if self._epoch_len is not None and index >= self._epoch_len:
                    epoch, index = epoch + 1, 0
                    self._open_epoch(epoch)
        except BaseException as exc:     # forwarded to the consumer, which re-raises it
            box.put(_Failure(exc))

    def _begin(self) -> None:
        self._halt()
        self._box.drain()
        self._release_iterator()
        # While a resume skip is pending, len(loader) reports only the remainder of the epoch;
        # measure the full epoch with the skip lifted and restore it for the iterator below.
        pending = getattr(self.sampler, "skip", 0)
        if pending:
            self.sampler.skip = 0
        try:
            full = _length(self.loader)
        finally:
            if pending:
                self.sampler.skip = pending
        self._epoch_len = full or self._epoch_len or None
        self._open_epoch(self._from[0])
        if self.threaded:
            self._box.stop.clear()
            self._thread = threading.Thread(target=self._produce, name="fmb200-batches", daemon=True)
            self._thread.start()
        else:
            try:
                self._stage_serial()
            except StopIteration:
                raise self._empty() from None

    def _stage_serial(self) -> None:
        try:
            batch = next(self._it)
        except StopIteration:
            self.epoch += 1
            self.batches = 0
            self._open_epoch(self.epoch)
            batch = next(self._it)
        payload, ev = self._copier.stage((batch["input_ids"], batch["labels"]))
        self._ahead = (payload, ev)

    # ---- consumer side
    def next(self):
        if not self.threaded:
            payload, ev = self._ahead
            out = self._copier.join(payload, ev)
            self.batches += 1
            self.stats["batches"] += 1
            self._stage_serial()
            return out
        t0 = time.perf_counter()
        item = self._box.get()
        waited = (time.perf_counter() - t0) * 1e3
        if isinstance(item, _Failure):
            self._halt()
            raise item.exc
        if item is _DONE:
            self._halt()
            if self.stats["batches"] == 0:
                raise self._empty()
            raise StopIteration
        st = self.stats
        st["wait_ms"] += waited
        st["max_wait_ms"] = max(st["max_wait_ms"], waited)
        st["stalled"] += waited > 1.0
        st["batches"] += 1
        self.epoch, self.batches = item.epoch, item.index + 1
        if item.epoch_len is not None and self.batches >= item.epoch_len:
            self.epoch, self.batches = item.epoch + 1, 0
        return self._copier.join(item.payload, item.event)

    __next__ = next

    def __iter__(self):
        return self

    # ---- control
    def resume(self, epoch: int, batches: int) -> None:
        self._halt()                 # the old producer must be gone before the sampler is touched
        self._box.drain()
        self._release_iterator()
        self.epoch, self.batches = epoch, batches
        self._from = (epoch, batches)
        self.sampler.skip = batches * int(getattr(self.loader, "batch_size", 0) or 0)
        self._begin()

    def report(self) -> dict:
        st = dict(self.stats)
        n = max(1, st["batches"])
        st["wait_ms_per_batch"] = round(st["wait_ms"] / n, 3)
        st["stall_ratio"] = round(st["stalled"] / n, 3)
        st["queued"] = self._box.q.qsize()
        return st

    def _empty(self) -> RuntimeError:
        return RuntimeError("BatchStream: the loader produced no batches (dataset smaller than "
                            f"batch_size={getattr(self.loader, 'batch_size', '?')} with drop_last=True?)")

    def _halt(self) -> None:
        th, self._thread = self._thread, None
        if th is not None:
            self._box.stop.set()
            th.join(timeout=10.0)
            if th.is_alive():  # pragma: no cover
                warn_once("batch prefetch thread did not stop within 10 s (blocked in dataset code); "
                          "it is a daemon and will not keep the process alive", key="batchstream-stop")

    def _release_iterator(self) -> None:
        it, self._it = self._it, None
        if it is not None:
            _finalize_iterator(it)

    def close(self) -> None:
        if self._closed:
            return
        self._halt()
        self._box.drain()
        self._release_iterator()
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


# ------------------------------------------------------------------------------ generic prefetcher
class _AsyncLoader:
    """One pass over any iterable of (nested) tensors, moved to ``device`` ahead of use."""

    def __init__(self, loader, device, depth: int = 2):
        self.loader = loader
        self.device = torch.device(device)
        self.depth = max(1, int(depth))
        self._copier = _Copier(self.device)
        self.stream = self._copier.stream
        self.stats = {"batches": 0, "wait_ms": 0.0, "stalled": 0, "max_wait_ms": 0.0}
        self._box = _Mailbox(self.depth)
        self._it = iter(loader)
        self._closed = False
        self._thread = threading.Thread(target=self._produce, name="fmb200-async-loader", daemon=True)
        self._thread.start()

    def _produce(self):
        _bind(self.device)
        try:
            while not self._box.stop.is_set():
                try:
                    batch = next(self._it)
                except StopIteration:
                    self._box.put(_DONE)
                    return
                payload, ev = self._copier.stage(batch)
                if not self._box.put(_Staged(payload, ev)):
                    return
        except BaseException as exc:
            self._box.put(_Failure(exc))

    def __iter__(self):
        return self

    def __next__(self):
        if self._closed:
            raise StopIteration
        t0 = time.perf_counter()
        item = self._box.get()
        waited = (time.perf_counter() - t0) * 1e3
        if isinstance(item, _Failure):
            self.close()
            raise item.exc
        if item is _DONE:
            self.close()
            raise StopIteration
        st = self.stats
        st["batches"] += 1
        st["wait_ms"] += waited
        st["max_wait_ms"] = max(st["max_wait_ms"], waited)
        st["stalled"] += waited > 1.0
        return self._copier.join(item.payload, item.event)

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        th, self._thread = self._thread, None
        if th is not None:
            self._box.stop.set()
            th.join(timeout=10.0)
        self._box.drain()
        it, self._it = self._it, None
        if it is not None:
            _finalize_iterator(it)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


def async_loader(loader, device, depth: int = 2):
    """``for batch in async_loader(loader, "cuda"):`` -- batches arrive on the device while the
    previous step is still running. One-shot: wrap the loader again for another epoch."""
    return _AsyncLoader(loader, device, depth=depth)


def build_loader(ds, micro_batch, ctx, seed=0, workers=0, shuffle=True, persistent_workers=None):
    """DataLoader + :class:`ResumableSampler` for ``ctx``'s data-parallel coordinate
    (``drop_last``; pinned memory on CUDA; persistent workers when ``workers > 0``)."""
    sampler = ResumableSampler(len(ds), ctx.dp_rank, ctx.dp_world, seed, shuffle)
    extra = {}
    if workers and workers > 0:
        extra = dict(num_workers=int(workers), prefetch_factor=2,
                     persistent_workers=True if persistent_workers is None else bool(persistent_workers))
    loader = DataLoader(ds, batch_size=micro_batch, sampler=sampler, drop_last=True,
                        pin_memory=ctx.device.type == "cuda", **extra)
    return loader, sampler
