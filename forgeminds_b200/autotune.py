"""Measure the cheap switches of a training step and report the fastest combination.

``autotune(target)`` times a baseline step of a :class:`~forgeminds_b200.forge.Forge` or
:class:`~forgeminds_b200.trainer.Trainer` and then a handful of variants (precision, fused kernels,
accumulation, rebuilt trainers for knobs that cannot be flipped on a live object); out-of-memory and
other failures are recorded as data, nothing is changed unless ``apply=True``. ``tune_batch_size``
sweeps micro-batch sizes by *per-sample* cost. ``autotune_kernels`` times the fused kernels of this
device with CUDA events. Interface of the reference's ``forgemind/autotune.py:48-372``.
"""
from __future__ import annotations

import contextlib
import json
import os
import statistics
import time
from dataclasses import dataclass, field

import torch

__all__ = ["Trial", "Report", "time_call", "apply_fast_defaults", "tune_batch_size", "autotune",
           "autotune_kernels"]


@dataclass
class Trial:
    label: str
    ok: bool = True
    ms: float = float("inf")
    note: str = ""
    oom: bool = False

    def __str__(self) -> str:
        status = "oom" if self.oom else ("ok" if self.ok else "fail")
        return f"{self.label:38s} {status:5s} {self.ms:9.2f} ms  {self.note}"


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
        return "\n".join([f"{'trial':38s} {'stat':5s} {'median':>9s}  note", *map(str, self.trials)])

    def speedup(self) -> float:
        best = self.best.get("ms")
        return self.baseline_ms / best if (self.baseline_ms and best) else 1.0

    def to_dict(self) -> dict:
        return {"device": self.device, "best": self.best, "baseline_ms": self.baseline_ms,
                "speedup": self.speedup(), "trials": [vars(t) for t in self.trials]}


def _is_oom(exc: BaseException) -> bool:
    if isinstance(exc, getattr(torch.cuda, "OutOfMemoryError", ())):
        return True
    return "out of memory" in str(exc).lower()


def time_call(fn, warmup: int = 2, repeats: int = 5, sync: bool = True) -> float:
    """Median wall time of ``fn()`` in milliseconds after ``warmup`` untimed calls."""
    wait = torch.cuda.synchronize if (sync and torch.cuda.is_available()) else (lambda: None)
    for _ in range(max(0, warmup)):
        fn()
    wait()
    samples = []
    for _ in range(max(1, repeats)):
        t0 = time.perf_counter()
        fn()
        wait()
        samples.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(samples)


def apply_fast_defaults(device=None, allow_tf32: bool = True, allocator: bool = True) -> dict:
    """Turn on the settings that are almost always free; returns what was changed."""
    changed = {}
    if allow_tf32:
        with contextlib.suppress(Exception):
            torch.backends.cuda.matmul.allow_tf32 = True
            torch.backends.cudnn.allow_tf32 = True
            torch.set_float32_matmul_precision("high")
            changed["tf32"] = True
    if torch.cuda.is_available():
        with contextlib.suppress(Exception):
            torch.backends.cudnn.benchmark = True
            changed["cudnn_benchmark"] = True
        if allocator and "PYTORCH_CUDA_ALLOC_CONF" not in os.environ:
            os.environ["PYTORCH_CUDA_ALLOC_CONF"] = "expandable_segments:True"
            changed["expandable_segments"] = "(set, takes effect on next process)"
    changed["threads"] = torch.get_num_threads()
    return changed


def tune_batch_size(step_fn, candidates=(1, 2, 4, 8, 16, 32), *, warmup: int = 1, repeats: int = 3,
                    min_gain: float = 0.02, footprint=None, report: "Report | None" = None):
    """Largest micro-batch that still lowers the cost per sample; stops at the first size without a
    gain of ``min_gain`` or at the first out-of-memory. Returns ``(size, ms_per_step)``."""
    report = report or Report()
    best = (None, float("inf"), float("inf"))       # size, ms, ms per sample
    for size in candidates:
        trial = Trial(label=f"micro_batch={size}")
        try:
            if footprint is not None:
                footprint(size)
            ms = time_call(lambda: step_fn(size), warmup=warmup, repeats=repeats)
        except BaseException as exc:      # noqa: BLE001 -- running out of memory is a result here
            if not _is_oom(exc):
                raise
            trial.ok, trial.oom, trial.note = False, True, "did not fit"
            report.add(trial)
            break
        per = ms / size
        better = best[0] is None or per < best[2] * (1.0 - min_gain)
        trial.ms, trial.note = ms, f"{per:.3f} ms/sample" + (", best so far" if better else ", no gain -> stop")
        report.add(trial)
        if not better:
            break
        best = (size, ms, per)
        if torch.cuda.is_available():
            with contextlib.suppress(Exception):
                torch.cuda.empty_cache()
    return (best[0] or candidates[0]), best[1]


def autotune(target, loader=None, *, build=None, budget_s: float = 60.0, apply: bool = False,
             precision: bool = True, accum: bool = True, compiled: bool = False, fused: bool = True,
             report: "Report | None" = None) -> Report:
    from .forge import Forge
    report = report or Report()
    report.device = str(getattr(target, "device", "cpu"))
    started = time.time()
    is_forge = isinstance(target, Forge)
    batch = next(iter(loader)) if (is_forge and loader is not None) else None

    def runner(obj):
        if is_forge and batch is not None:
            return lambda: obj.step(batch)
        return lambda: obj.train_step()

    def measure(label, before=None, after=None, note="", obj=None):
        if time.time() - started > budget_s:
            report.add(Trial(label, ok=False, note="skipped: budget"))
            return float("inf")
        try:
            if before:
                before()
            trial = Trial(label, ms=time_call(runner(obj or target), warmup=1, repeats=3), note=note)
        except BaseException as exc:      # noqa: BLE001
            trial = Trial(label, ok=False, oom=_is_oom(exc), note=str(exc).replace("\n", " ")[:60])
        finally:
            if after:
                after()
        report.add(trial)
        return trial.ms

    def override(**values):
        saved = {}

        def before():
            for k, v in values.items():
                saved[k] = getattr(target, k)
                setattr(target, k, v)

        def after():
            for k, v in saved.items():
                setattr(target, k, v)
        return before, after

    report.baseline_ms = best_ms = measure("baseline")
    best: dict = {}

    if is_forge:
        if precision and report.device.startswith("cuda"):
            for name, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
                ms = measure(f"precision={name}", *override(precision=name, amp_dtype=dt))
                if ms < best_ms:
                    best_ms, best = ms, {"precision": name}
        if fused:
            from .kernels import available
            if available():
                from .kernels.apply import enable, revert
                memo = {}

                def fuse():
                    memo["already"] = any(getattr(m, "_fm_norm", False) or getattr(m, "_fm_mlp", False)
                                          for m in target.raw_model.modules())
                    enable(target.raw_model)

                def unfuse():
                    if not memo.get("already"):
                        revert(target.raw_model)
                ms = measure("fused_kernels=on", fuse, unfuse, note="rmsnorm+swiglu kernels")
                if ms < best_ms:
                    best_ms, best = ms, {"fused_ops": True}
        if accum and getattr(target, "accum", 1) > 1:
            ms = measure("accum=1 (per-micro-batch cost)", *override(accum=1, micro=0))
            if ms and ms < best_ms:
                best_ms, best = ms, {"accum": 1}

    if build is not None:
        variants = ([("bf16", {"bf16": True})] if precision else []) + [("ac=full", {"ac": "full"})]
        if compiled:
            variants.append(("compile", {"compile": True}))
        for label, over in variants:
            try:
                rebuilt = build(**over)
            except BaseException as exc:      # noqa: BLE001
                report.add(Trial(f"build {label}", ok=False, note=str(exc)[:60]))
                continue
            ms = measure(f"{label} (rebuilt)", note=str(over), obj=rebuilt)
            if ms < best_ms:
                best_ms, best = ms, dict(over)
            with contextlib.suppress(Exception):
                if hasattr(rebuilt, "close"):
                    rebuilt.close()
            del rebuilt
            if torch.cuda.is_available():
                with contextlib.suppress(Exception):
                    torch.cuda.empty_cache()

    report.best = dict(best, ms=best_ms)
    if apply and best:
        for k, v in best.items():
            setattr(target, k, v)
    return report


def autotune_kernels(candidates=None, iters: int = 20, cache: bool = True) -> dict:
    """Time the fused kernels on this GPU (``{"skipped": ...}`` without one). The kernels have no
    launch parameters to sweep; the numbers are a health check and a baseline for comparisons."""
    from . import kernels
    if not kernels.available():
        return {"skipped": "needs a CUDA device of compute capability 10 and the native extension",
                "device": str(torch.device("cpu"))}
    d = 4096
    x = torch.randn(8192, d, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(d, device="cuda")
    gu = torch.randn(8192, 2 * 11008 // 16 * 16, device="cuda", dtype=torch.bfloat16)
    out = {}
    for name, fn in (("rms_norm", lambda: kernels.rms_norm(x, w, 1e-6)),
                     ("swiglu_split", lambda: kernels.swiglu_split(gu))):
        try:
            out[name] = {"ms": time_call(fn, warmup=3, repeats=iters)}
        except Exception as exc:
            out[name] = {"ms": float("nan"), "note": str(exc)[:80]}
    out["device"] = torch.cuda.get_device_name()
    return out


def _main(argv=None) -> int:
    import argparse
    from .forge import Forge
    from .models import GPT, GPTConfig
    ap = argparse.ArgumentParser(description="autotune a training step on this device")
    ap.add_argument("--preset", default="tiny")
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--budget", type=float, default=60.0)
    ap.add_argument("--apply", action="store_true")
    ap.add_argument("--kernels", action="store_true")
    a = ap.parse_args(argv)
    if a.kernels:
        print(json.dumps(autotune_kernels(), indent=1))
        return 0
    dim = {"tiny": 128, "small": 256, "medium": 512}.get(a.preset, 128)
    mc = GPTConfig(vocab_size=512, dim=dim, n_layers=4, n_heads=max(2, dim // 32), n_kv_heads=max(1, dim // 64),
                   max_seq=a.seq)
    forge = Forge(GPT(mc), None, precision="bf16" if torch.cuda.is_available() else "fp32",
                  loss_fn=lambda out, b: out[0] if isinstance(out, (tuple, list)) else out)
    x = torch.randint(0, mc.vocab_size, (a.micro_batch, a.seq))
    y = torch.randint(0, mc.vocab_size, (a.micro_batch, a.seq))
    print("fast defaults:", apply_fast_defaults())
    rep = autotune(forge, [(x, y)], budget_s=a.budget, apply=a.apply)
    print(rep.table())
    print(f"baseline {rep.baseline_ms:.2f} ms -> best {rep.best.get('ms', 0):.2f} ms ({rep.speedup():.2f}x) {rep.best}")
    return 0


if __name__ == "__main__":  # pragma: no cover
    raise SystemExit(_main())
