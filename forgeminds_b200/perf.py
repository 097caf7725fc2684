"""Host-sync auditing and small performance helpers.

The training loops in this library are built around a budget of one host<->device
synchronisation per optimizer step. :func:`count_host_syncs` makes that budget testable: while
the context is open, every tensor method that forces the host to wait for the device
(``item``, ``tolist``, ``numpy``, ``cpu``, ``__float__``/``__int__``/``__bool__``) and the
explicit waits (``torch.cuda.synchronize``, ``Stream.synchronize``, ``Event.synchronize``) are
counted and attributed to the calling module. Same contract as the reference's
``forgemind/perf.py:44-180``.
"""
from __future__ import annotations

import contextlib
import os
import sys
import threading
import warnings

import torch

__all__ = ["count_host_syncs", "host_syncs", "HostSyncCounter", "warn_once", "enable_fast_math",
           "pinned_pool", "DeviceTimer"]

_PKG = __name__.split(".")[0]
_TENSOR_READS = ("item", "tolist", "numpy", "cpu", "__float__", "__int__", "__bool__")


class HostSyncCounter:
    """Tally of host-blocking reads seen while a :func:`count_host_syncs` block was open."""

    def __init__(self, capture_stack: bool = True, stack_limit: int = 4):
        self.count = 0
        self.own = 0          # raised from inside this package
        self.external = 0     # raised from torch internals or user code
        self.capture_stack = capture_stack
        self.stack_limit = stack_limit
        self.sites: dict = {}

    def record(self, label: str, frame) -> None:
        self.count += 1
        module = frame.f_globals.get("__name__", "") if frame is not None else ""
        if module == _PKG or module.startswith(_PKG + "."):
            self.own += 1
        else:
            self.external += 1
        if self.capture_stack and frame is not None:
            code = frame.f_code
            where = f"{os.path.basename(code.co_filename)}:{frame.f_lineno} {code.co_name} [{label}]"
            self.sites[where] = self.sites.get(where, 0) + 1

    def report(self) -> str:
        head = f"{self.count} host sync(s): {self.own} from {_PKG}, {self.external} from elsewhere"
        top = sorted(self.sites.items(), key=lambda kv: kv[1], reverse=True)[: self.stack_limit]
        return "\n".join([head] + [f"  {n:>4}x {site}" for site, n in top])


class _Audit:
    """Installs and removes the counting wrappers; shared by all open counters."""

    def __init__(self):
        self.lock = threading.RLock()
        self.active: list = []
        self.saved: list = []        # (owner, attribute, original)
        self.total = 0
        self.count_cpu = False

    def _emit(self, label):
        self.total += 1
        frame = sys._getframe(2)
        for c in tuple(self.active):
            c.record(label, frame)

    def _wrap_tensor_method(self, name):
        original = getattr(torch.Tensor, name)
        audit = self

        def counted(tensor, *a, **k):
            if tensor.is_cuda or audit.count_cpu:
                audit._emit(name)
            return original(tensor, *a, **k)
        counted._fmb_counted = True
        self.saved.append((torch.Tensor, name, original))
        setattr(torch.Tensor, name, counted)

    def _wrap_wait(self, owner, label):
        original = getattr(owner, "synchronize", None)
        if original is None or getattr(original, "_fmb_counted", False):
            return
        audit = self

        def counted(*a, **k):
            if torch.cuda.is_available() or audit.count_cpu:
                audit._emit(label)
            return original(*a, **k)
        counted._fmb_counted = True
        self.saved.append((owner, "synchronize", original))
        setattr(owner, "synchronize", counted)

    def install(self):
        if self.saved:
            return
        for name in _TENSOR_READS:
            if hasattr(torch.Tensor, name):
                self._wrap_tensor_method(name)
        self._wrap_wait(torch.cuda, "cuda.synchronize")
        self._wrap_wait(torch.cuda.Stream, "Stream.synchronize")
        self._wrap_wait(torch.cuda.Event, "Event.synchronize")

    def remove(self):
        for owner, name, original in reversed(self.saved):
            setattr(owner, name, original)
        self.saved.clear()


_AUDIT = _Audit()


@contextlib.contextmanager
def count_host_syncs(capture_stack: bool = True, count_cpu: bool = False):
    """Yield a :class:`HostSyncCounter`. Reads of CPU tensors are ignored unless ``count_cpu`` is
    set, which lets a GPU-less test suite check the number and place of host reads."""
    counter = HostSyncCounter(capture_stack)
    with _AUDIT.lock:
        _AUDIT.install()
        previous = _AUDIT.count_cpu
        _AUDIT.count_cpu = bool(count_cpu)
        _AUDIT.active.append(counter)
    try:
        yield counter
    finally:
        with _AUDIT.lock:
            _AUDIT.active.remove(counter)
            _AUDIT.count_cpu = previous
            if not _AUDIT.active:
                _AUDIT.remove()


def host_syncs() -> int:
    """Number of host-blocking reads counted so far in this process (0 if never audited)."""
    return _AUDIT.total


# ------------------------------------------------------------------------------ misc helpers
_seen: set = set()
_seen_lock = threading.Lock()


def warn_once(msg: str, key: str | None = None) -> None:
    tag = msg if key is None else key
    with _seen_lock:
        if tag in _seen:
            return
        _seen.add(tag)
    warnings.warn(msg, stacklevel=3)


def enable_fast_math(enabled: bool = True) -> None:
    """TF32 for the fp32 leftovers and cuDNN autotuning; nothing to do without a GPU."""
    if not torch.cuda.is_available():
        return
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cudnn.benchmark = True
    if enabled:
        with contextlib.suppress(Exception):
            torch.set_float32_matmul_precision("high")


class _PinnedPool:
    """Free lists of pinned host buffers keyed by (shape, dtype).

    ``get`` reuses a returned buffer of the same key or allocates; ``put`` hands a buffer back.
    A buffer must only be returned after the copy that reads it has been ordered on a stream.
    """

    def __init__(self, pin: bool = True):
        self.pin = bool(pin) and torch.cuda.is_available()
        self.hits = 0
        self.misses = 0
        self._shelves: dict = {}

    def get(self, shape, dtype) -> torch.Tensor:
        shelf = self._shelves.get((tuple(shape), dtype))
        if shelf:
            self.hits += 1
            return shelf.pop()
        self.misses += 1
        return torch.empty(tuple(shape), dtype=dtype, device="cpu", pin_memory=self.pin)

    def put(self, buf: torch.Tensor) -> None:
        self._shelves.setdefault((tuple(buf.shape), buf.dtype), []).append(buf)

    def clear(self) -> None:
        self._shelves.clear()


def pinned_pool(pin: bool = True) -> _PinnedPool:
    return _PinnedPool(pin)


class DeviceTimer:
    """CUDA-event stopwatch on the current stream; falls back to the host clock on CPU.

    ``elapsed_ms`` synchronises on the stop event, so call it outside the region under audit.
    """

    def __init__(self, device=None):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._t0 = self._t1 = None

    def start(self):
        if self.cuda:
            self._t0 = torch.cuda.Event(enable_timing=True)
            self._t1 = torch.cuda.Event(enable_timing=True)
            self._t0.record()
        else:
            import time
            self._t0 = time.perf_counter()
        return self

    def stop(self):
        if self.cuda:
            self._t1.record()
        else:
            import time
            self._t1 = time.perf_counter()
        return self

    def elapsed_ms(self) -> float:
        if self.cuda:
            self._t1.synchronize()
            return float(self._t0.elapsed_time(self._t1))
        return (self._t1 - self._t0) * 1e3
