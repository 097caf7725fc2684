"""Loader and autograd wrappers for the sm_100a kernels.

``native()`` returns the compiled extension (``forgeminds_b200/_C.so``, built in-tree by
``forgeminds_b200.csrc.build``). On a machine with a CUDA device a missing extension is an error,
not a silent fall-back: :func:`require` raises with the build command. On CPU the pure-PyTorch
paths in :mod:`forgeminds_b200.kernels.reference` are used instead.
"""
from __future__ import annotations

import importlib
import os
import threading

import torch

_lock = threading.Lock()
_mod = None
_err: Exception | None = None


def native():
    """The extension module, or ``None`` if it cannot be imported."""
    global _mod, _err
    if _mod is not None or _err is not None:
        return _mod
    with _lock:
        if _mod is None and _err is None:
            try:
                # FORGEMINDS_DEBUG_SO=1: the build with bounds checks on every peer-memory access
                # (python -m forgeminds_b200.csrc.build --debug-bounds)
                name = "_C_debug" if os.environ.get("FORGEMINDS_DEBUG_SO") == "1" else "_C"
                _mod = importlib.import_module(f"forgeminds_b200.{name}")
            except Exception as exc:  # missing file, wrong ABI, no libcudart ...
                _err = exc
    return _mod


def available() -> bool:
    """True when the kernels can run here: a CUDA device of compute capability 10.x and the extension."""
    if not torch.cuda.is_available():
        return False
    try:
        major, _ = torch.cuda.get_device_capability()
    except Exception:
        return False
    return major == 10 and native() is not None


def require():
    """Extension module or a loud error (used by every GPU code path)."""
    mod = native()
    if mod is None:
        raise RuntimeError(
            "forgeminds_b200: the native extension forgeminds_b200/_C.so is missing or failed to load "
            f"({_err!r}). Build it with `python -m forgeminds_b200.csrc.build`.")
    return mod


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels set when one of their bounded waits runs out."""
    key = torch.device(device)
    if key.type == "cuda" and key.index is None:          # "cuda" and "cuda:0" must name the same word
        key = torch.device("cuda", torch.cuda.current_device())
    word = _status.get(key)
    if word is None:
        word = _status[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return word


_status: dict = {}


class CommTimeout(RuntimeError):
    """A device-side wait gave up; the status word holds the error code."""


class BoundsError(RuntimeError):
    """Debug build only: a kernel was about to touch memory outside every registered buffer (code 7);
    the access was skipped."""


class EPOverflow(RuntimeError):
    """An expert-parallel layer routed more rows to one rank than its dispatch buffers hold
    (``parallel.ep_slot_factor``, code 8); the rows beyond were left out and the step must not be trusted."""


ERR_EP_OVERFLOW = 8


def register_buffer(t_or_ptr, nbytes: int | None = None, device=None) -> None:
    """Debug build: add a buffer (a tensor, or an address and a length) to the table that the checked
    peer-memory accesses are validated against. No-op in the normal build."""
    mod = native()
    if mod is None or not hasattr(mod, "debug_bounds") or not mod.debug_bounds():
        return
    if torch.is_tensor(t_or_ptr):
        base, nbytes, device = t_or_ptr.data_ptr(), t_or_ptr.numel() * t_or_ptr.element_size(), t_or_ptr.device
    else:
        base = int(t_or_ptr)
    if nbytes:
        mod.debug_register(base, int(nbytes), status_word(device))


def check_status(device, sync_value: int | None = None) -> None:
    """Raise :class:`CommTimeout` if a kernel reported a timed-out wait. ``sync_value`` lets a
    caller pass a value it already brought to the host so that no extra sync is paid."""
    code = int(status_word(device).item()) if sync_value is None else int(sync_value)
    if code:
        status_word(device).zero_()
        if code == 7:
            raise BoundsError("forgeminds_b200: a kernel of the bounds-checked build skipped an access outside "
                              "every registered buffer (code 7)")
        if code == ERR_EP_OVERFLOW:
            raise EPOverflow("forgeminds_b200: an expert-parallel layer routed more rows to one rank than "
                             "parallel.ep_slot_factor provides room for (code 8): raise the factor or set it to 0")
        raise CommTimeout(f"forgeminds_b200: a kernel wait timed out (code {code})")
