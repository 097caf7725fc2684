"""Step audit: host reads per step, kernel launches per step, kernel time against step time and the top kernels.

    python -m forgeminds_b200.cli audit --preset tiny --steps 5
    python -m forgeminds_b200.cli audit --preset medium --seq 2048 --micro-batch 4 --grad-accum 4 --ac selective --budget 1

Exit code 3 when the training loop reads the device more than ``--budget`` times per optimizer step
(reads made inside PyTorch itself are listed separately and do not count). Covers what the
reference's ``tools/profile_audit.py`` reports (profiler table, host-read attribution); the
graph-break part of that tool has no counterpart here because no tracing compiler is on the hot path.
"""
from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> int:
    from .. import GPT, GPTConfig, SyntheticLM, Trainer, cleanup, ops
    from ..perf import count_host_syncs
    from .bench import PRESETS, build_config, parse as bench_parse
    p = argparse.ArgumentParser(prog="forgeminds_b200.cli audit", add_help=True)
    p.add_argument("--budget", type=float, default=1.0, help="allowed host reads per optimizer step")
    p.add_argument("--top", type=int, default=12)
    p.add_argument("--json", dest="audit_json", default=None)
    own, rest = p.parse_known_args(argv)
    a = bench_parse(rest)
    cfg = build_config(a)
    mc = GPTConfig(vocab_size=32000, max_seq=a.seq, n_experts=a.experts if a.moe else 0, top_k=a.top_k,
                   ffn_hidden=a.ffn_hidden or None, capacity_factor=a.capacity_factor, **PRESETS[a.preset])
    ds = SyntheticLM(mc.vocab_size, a.seq, n=max(256, a.micro_batch * a.grad_accum * (a.warmup + a.steps) * 2))
    tr = Trainer(lambda ctx: GPT(mc), cfg, ds, micro_batch=a.micro_batch)
    on_gpu = tr.ctx.device.type == "cuda"
    for _ in range(a.warmup):
        tr.train_step()
    native = ops.native() if on_gpu else None
    launches0 = native.launch_count() if native is not None else 0
    with count_host_syncs(capture_stack=True, count_cpu=not on_gpu) as counter:
        for _ in range(a.steps):
            tr.train_step()
    launches = (native.launch_count() - launches0) / a.steps if native is not None else 0.0
    report = {
        "engine": "native" if tr.store is not None else "library",
        "host_reads_per_step": counter.own / a.steps,
        "host_reads_inside_torch_per_step": counter.external / a.steps,
        "library_kernel_launches_per_step": launches,
        "budget": own.budget,
    }
    if on_gpu:
        from torch.profiler import ProfilerActivity, profile
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            t0 = torch.cuda.Event(enable_timing=True)
            t1 = torch.cuda.Event(enable_timing=True)
            t0.record()
            tr.train_step()
            t1.record()
            torch.cuda.synchronize()
        events = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
        busy_ms = sum(e.device_time for e in events) / 1e3
        report["step_ms_under_profiler"] = t0.elapsed_time(t1)
        # kernels launched with programmatic dependent launch start (and are timed) while their
        # predecessor drains, so this ratio can exceed 1; well below 1 means the GPU waits for the host
        report["kernel_time_over_step_time"] = busy_ms / max(t0.elapsed_time(t1), 1e-9)
        by_name: dict = {}
        for e in events:
            slot = by_name.setdefault(e.name[:80], [0, 0.0])
            slot[0] += 1
            slot[1] += e.device_time / 1e3
        report["top_kernels"] = [dict(name=k, calls=n, ms=round(ms, 3))
                                 for k, (n, ms) in sorted(by_name.items(), key=lambda kv: -kv[1][1])[:own.top]]
    tr.close()
    if tr.ctx.rank == 0:
        print("=== forgeminds_b200 step audit ===")
        for k, v in report.items():
            if k != "top_kernels":
                print(f"{k:>36}: {v}")
        for row in report.get("top_kernels", []):
            print(f"{row['ms']:10.3f} ms  x{row['calls']:<5d} {row['name']}")
        if counter.own:
            print(counter.report())
        if own.audit_json:
            with open(own.audit_json, "w") as f:
                json.dump(report, f, indent=2)
    cleanup()
    return 3 if report["host_reads_per_step"] > own.budget + 1e-9 else 0


if __name__ == "__main__":
    raise SystemExit(main())
