"""Try the cheap knobs of a training step, time each, and say which combination is fastest.

Nothing here guesses: every candidate is run for a few steps and timed; a candidate that runs out of
memory or raises is written down as a result, not propagated. Entry points (the reference's
``forgemind/autotune.py:48-372``):

* :func:`autotune` -- baseline plus variants of a live :class:`~forgeminds_b200.forge.Forge` (autocast
  dtype, fused kernels patched in, accumulation off) and of trainers rebuilt through ``build(**knobs)``
  for settings that cannot be flipped on a live object; stays within ``budget_s`` seconds;
* :func:`tune_batch_size` -- grows the micro-batch while the cost *per sample* keeps falling;
* :func:`apply_fast_defaults` -- the process-wide switches that are free on this hardware;
* :func:`autotune_kernels` -- device timings of the fused kernels (a health check: they have no launch
  parameters to sweep);
* ``python -m forgeminds_b200.autotune`` -- the same on a small GPT from the command line.
"""
from __future__ import annotations

import gc
import json
import os
import statistics
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Optional

import torch

__all__ = ["Trial", "Report", "time_call", "apply_fast_defaults", "tune_batch_size", "autotune",
           "autotune_kernels"]

INF = float("inf")


@dataclass
class Trial:
    """One timed candidate. ``ok`` is false when it did not run to the end; ``oom`` says why, if memory."""
    label: str
    ok: bool = True
    ms: float = INF
    note: str = ""
    oom: bool = False

    @property
    def outcome(self) -> str:
        if self.oom:
            return "OOM"
        return "done" if self.ok else "error"

    def row(self, width: int) -> str:
        took = f"{self.ms:10.3f}" if self.ms < INF else f"{'-':>10s}"
        return f"{self.label:<{width}s}  {self.outcome:<5s}  {took}  {self.note}".rstrip()


@dataclass
class Report:
    device: str = ""
    trials: list = field(default_factory=list)
    best: dict = field(default_factory=dict)
    baseline_ms: float = 0.0

    def add(self, trial: Trial) -> Trial:
        self.trials.append(trial)
        return trial

    def table(self) -> str:
        width = max([len(t.label) for t in self.trials] + [9])
        head = f"{'candidate':<{width}s}  {'end':<5s}  {'median ms':>10s}  remarks"
        return "\n".join([head, "-" * len(head)] + [t.row(width) for t in self.trials])

    def speedup(self) -> float:
        winner = self.best.get("ms")
        if not winner or not self.baseline_ms or winner == INF or self.baseline_ms == INF:
            return 1.0
        return self.baseline_ms / winner

    def to_dict(self) -> dict:
        return {"device": self.device, "baseline_ms": self.baseline_ms, "best": dict(self.best),
                "speedup": self.speedup(), "trials": [asdict(t) for t in self.trials]}


def _out_of_memory(err: BaseException) -> bool:
    oom_type = getattr(torch.cuda, "OutOfMemoryError", None)
    if oom_type is not None and isinstance(err, oom_type):
        return True
    return "out of memory" in f"{err}".lower()


def _drain_gpu() -> None:
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def _free_cached() -> None:
    gc.collect()
    if torch.cuda.is_available():
        try:
            torch.cuda.empty_cache()
        except RuntimeError:
            pass


def time_call(fn: Callable[[], object], warmup: int = 2, repeats: int = 5, sync: bool = True) -> float:
    """Milliseconds per call of ``fn`` (median of ``repeats`` calls, after ``warmup`` calls that are not
    timed). With ``sync`` every timed call ends with a device synchronisation, so the figure includes the
    GPU work the call enqueued."""
    settle = _drain_gpu if sync else (lambda: None)
    for _ in range(max(0, int(warmup))):
        fn()
    settle()
    laps = []
    for _ in range(max(1, int(repeats))):
        begin = time.perf_counter()
        fn()
        settle()
        laps.append(1e3 * (time.perf_counter() - begin))
    return statistics.median(laps)


def apply_fast_defaults(device=None, allow_tf32: bool = True, allocator: bool = True) -> dict:
    """Switch on what costs nothing: TF32 for stray fp32 matmuls, cuDNN autotuning, and (for processes
    started after this one) the expandable-segments allocator. Returns a dict of what was touched."""
    did: dict = {}
    if allow_tf32:
        try:
            torch.set_float32_matmul_precision("high")
            torch.backends.cudnn.allow_tf32 = True
            torch.backends.cuda.matmul.allow_tf32 = True
            did["tf32"] = True
        except (RuntimeError, AttributeError):
            did["tf32"] = False
    on_gpu = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
    if on_gpu:
        torch.backends.cudnn.benchmark = True
        did["cudnn_benchmark"] = True
        if allocator:
            if os.environ.get("PYTORCH_CUDA_ALLOC_CONF"):
                did["allocator"] = "left as configured: " + os.environ["PYTORCH_CUDA_ALLOC_CONF"]
            else:
                os.environ["PYTORCH_CUDA_ALLOC_CONF"] = "expandable_segments:True"
                did["allocator"] = "expandable_segments:True exported; child processes and the next run use it"
    did["cpu_threads"] = torch.get_num_threads()
    return did


def tune_batch_size(step_fn: Callable[[int], object], candidates=(1, 2, 4, 8, 16, 32), *, warmup: int = 1,
                    repeats: int = 3, min_gain: float = 0.02, footprint=None,
                    report: Optional[Report] = None):
    """Walk up ``candidates`` while a bigger micro-batch is cheaper per sample by at least ``min_gain``.

    ``step_fn(size)`` runs one step at that size; ``footprint(size)``, when given, is called first (allocate
    the batch there, so that a size that cannot even be staged counts as not fitting). The walk ends at
    the first size that does not fit in memory or brings no gain. Returns ``(size, ms per step)`` of the
    winner; other exceptions propagate."""
    log = report if report is not None else Report()
    winner_size, winner_ms, winner_unit = None, INF, INF
    for size in candidates:
        entry = Trial(label=f"micro_batch={size}")
        log.add(entry)
        try:
            if footprint is not None:
                footprint(size)
            took = time_call(lambda: step_fn(size), warmup=warmup, repeats=repeats)
        except BaseException as err:  # noqa: BLE001 - an allocation failure is an answer, anything else is a bug
            if not _out_of_memory(err):
                raise
            entry.ok, entry.oom, entry.note = False, True, "does not fit in device memory; search ends"
            break
        unit = took / size
        entry.ms = took
        improved = winner_size is None or unit < (1.0 - min_gain) * winner_unit
        entry.note = f"{unit:.3f} ms per sample" + ("" if improved else f" (less than {min_gain:.0%} better; search ends)")
        if not improved:
            break
        winner_size, winner_ms, winner_unit = size, took, unit
        _free_cached()
    if winner_size is None:
        return candidates[0], winner_ms
    return winner_size, winner_ms


class _Knob:
    """A reversible change to a live object: attribute overrides and/or a pair of callbacks."""

    def __init__(self, label: str, result: dict, target=None, attrs: Optional[dict] = None, enter=None, leave=None,
                 note: str = ""):
        self.label, self.result, self.note = label, result, note
        self.target, self.attrs, self.enter, self.leave = target, attrs or {}, enter, leave
        self._old: dict = {}

    def __enter__(self):
        for name, value in self.attrs.items():
            self._old[name] = getattr(self.target, name)
            setattr(self.target, name, value)
        if self.enter is not None:
            self.enter()
        return self

    def __exit__(self, *exc):
        if self.leave is not None:
            self.leave()
        for name, value in self._old.items():
            setattr(self.target, name, value)
        self._old.clear()
        return False


def _forge_knobs(forge, precision: bool, fused: bool, accum: bool) -> list:
    knobs = []
    if precision and forge.device.type == "cuda":
        from .forge import _Amp
        for name in ("bf16", "fp16"):
            if name != forge.precision:
                knobs.append(_Knob(f"precision={name}", {"precision": name}, forge,
                                   {"precision": name, "amp": _Amp(name, forge.device)}))
    if fused:
        from . import kernels
        if kernels.available():
            from .kernels.apply import enable, revert
            patched_before = any(getattr(m, "_fm_norm", False) or getattr(m, "_fm_mlp", False)
                                 for m in forge.raw_model.modules())
            knobs.append(_Knob("fused_kernels=on", {"fused_ops": True}, note="RMSNorm and SwiGLU modules call the kernels",
                               enter=lambda: enable(forge.raw_model),
                               leave=(lambda: None) if patched_before else (lambda: revert(forge.raw_model))))
    if accum and forge.accum > 1:
        from .forge import _Window
        knobs.append(_Knob("accum=1", {"accum": 1}, forge, {"accum": 1, "window": _Window()},
                           note="cost of one micro-batch plus an update"))
    return knobs


def autotune(target, loader=None, *, build=None, budget_s: float = 60.0, apply: bool = False,
             precision: bool = True, accum: bool = True, compiled: bool = False, fused: bool = True,
             report: Optional[Report] = None) -> Report:
    """Time ``target`` (a ``Forge`` fed from ``loader``, or anything with ``train_step()``) as it is and
    under each applicable variant; ``build(**knobs)`` returns a fresh trainer for variants that need one
    (``bf16``, ``ac="full"``, ``compile`` when ``compiled``). Candidates that would start after
    ``budget_s`` seconds are listed as skipped. ``apply=True`` leaves the winning attribute values on
    ``target``. The winner and its time are in ``report.best``."""
    from .forge import Forge
    rep = report if report is not None else Report()
    rep.device = str(getattr(target, "device", "cpu"))
    deadline = time.monotonic() + float(budget_s)
    live_forge = isinstance(target, Forge)
    sample = next(iter(loader)) if (live_forge and loader is not None) else None

    def one_step(obj):
        if isinstance(obj, Forge) and sample is not None:
            return lambda: obj.step(sample)
        return obj.train_step

    def clock(label: str, obj, note: str = "", scope=None) -> float:
        entry = rep.add(Trial(label, note=note))
        if time.monotonic() > deadline:
            entry.ok, entry.note = False, "not run: time budget used up"
            return INF
        try:
            if scope is not None:
                with scope:
                    entry.ms = time_call(one_step(obj), warmup=1, repeats=3)
            else:
                entry.ms = time_call(one_step(obj), warmup=1, repeats=3)
        except BaseException as err:  # noqa: BLE001 - failures are rows of the report
            entry.ok, entry.oom = False, _out_of_memory(err)
            entry.note = " ".join(f"{type(err).__name__}: {err}".split())[:70]
            _free_cached()
        return entry.ms

    rep.baseline_ms = clock("baseline", target)
    lead_ms, lead = rep.baseline_ms, {}

    if live_forge:
        for knob in _forge_knobs(target, precision, fused, accum):
            took = clock(knob.label, target, knob.note, scope=knob)
            if took < lead_ms:
                lead_ms, lead = took, dict(knob.result)

    if build is not None:
        rebuilds = []
        if precision:
            rebuilds.append({"bf16": True})
        rebuilds.append({"ac": "full"})
        if compiled:
            rebuilds.append({"compile": True})
        for knobs in rebuilds:
            label = "rebuilt with " + ", ".join(f"{k}={v}" for k, v in knobs.items())
            try:
                fresh = build(**knobs)
            except BaseException as err:  # noqa: BLE001
                rep.add(Trial(label, ok=False, oom=_out_of_memory(err),
                              note=" ".join(f"build failed: {err}".split())[:70]))
                continue
            took = clock(label, fresh)
            if took < lead_ms:
                lead_ms, lead = took, dict(knobs)
            closer = getattr(fresh, "close", None)
            if callable(closer):
                try:
                    closer()
                except Exception:  # noqa: BLE001
                    pass
            del fresh
            _free_cached()

    rep.best = {**lead, "ms": lead_ms}
    if apply:
        for name, value in lead.items():
            if name == "precision" and live_forge:
                from .forge import _Amp
                target.amp = _Amp(value, target.device)
            setattr(target, name, value)
    return rep


def autotune_kernels(candidates=None, iters: int = 20, cache: bool = True) -> dict:
    """Device timings (ms, fwd only) of the element-wise kernels at a 4096-wide model's shapes, or
    ``{"skipped": reason}`` where they cannot run. ``candidates`` / ``cache`` are accepted for
    compatibility: these kernels size their launch from the row width, there is nothing to search."""
    from . import kernels
    if not kernels.available():
        return {"skipped": "the sm_100a kernels need a compute-capability-10 GPU and the built extension",
                "device": "cpu" if not torch.cuda.is_available() else torch.cuda.get_device_name()}
    rows, width, hidden = 8192, 4096, 11008
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(rows, width, device="cuda", dtype=torch.bfloat16, generator=gen)
    delta = torch.randn(rows, width, device="cuda", dtype=torch.bfloat16, generator=gen)
    gain = torch.ones(width, device="cuda")
    gate_up = torch.randn(rows, 2 * hidden, device="cuda", dtype=torch.bfloat16, generator=gen)
    cases = {
        "rms_norm": lambda: kernels.rms_norm(x, gain, 1e-6),
        "add_rms_norm": lambda: kernels.add_rms_norm(x, delta, gain, 1e-6),
        "swiglu_split": lambda: kernels.swiglu_split(gate_up),
    }
    result = {"device": torch.cuda.get_device_name(), "shapes": {"rows": rows, "dim": width, "hidden": hidden}}
    for name, call in cases.items():
        try:
            result[name] = {"ms": time_call(call, warmup=3, repeats=iters)}
        except Exception as err:  # noqa: BLE001
            result[name] = {"ms": float("nan"), "note": f"{err}"[:80]}
    return result


def _main(argv=None) -> int:
    import argparse
    from .forge import Forge
    from .models import GPT, GPTConfig
    ap = argparse.ArgumentParser(prog="python -m forgeminds_b200.autotune",
                                 description="Time a small GPT training step under the cheap knobs of this library.")
    ap.add_argument("--preset", default="tiny", choices=["tiny", "small", "medium"])
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--budget", type=float, default=60.0, help="seconds")
    ap.add_argument("--apply", action="store_true", help="keep the winning settings on the Forge object")
    ap.add_argument("--kernels", action="store_true", help="only time the fused kernels")
    opts = ap.parse_args(argv)
    if opts.kernels:
        print(json.dumps(autotune_kernels(), indent=2))
        return 0
    width = {"tiny": 128, "small": 256, "medium": 512}[opts.preset]
    mc = GPTConfig(vocab_size=512, dim=width, n_layers=4, n_heads=max(2, width // 32), n_kv_heads=max(1, width // 64),
                   max_seq=opts.seq)
    on_gpu = torch.cuda.is_available()
    forge = Forge(GPT(mc), None, precision="bf16" if on_gpu else "fp32", quiet=True, async_batches=False,
                  forward_fn=lambda m, b: m(b[0], labels=b[1]))
    gen = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, mc.vocab_size, (opts.micro_batch, opts.seq + 1), generator=gen)
    print("process defaults:", json.dumps(apply_fast_defaults()))
    rep = autotune(forge, [(tokens[:, :-1], tokens[:, 1:])], budget_s=opts.budget, apply=opts.apply)
    print(rep.table())
    print(f"baseline {rep.baseline_ms:.2f} ms; fastest {rep.best['ms']:.2f} ms "
          f"({rep.speedup():.2f}x) with {({k: v for k, v in rep.best.items() if k != 'ms'}) or 'the baseline settings'}")
    return 0


if __name__ == "__main__":  # pragma: no cover
    raise SystemExit(_main())
