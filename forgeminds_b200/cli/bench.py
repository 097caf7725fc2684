"""Training benchmark of a GPT preset through :class:`forgeminds_b200.Trainer`.

    python -m forgeminds_b200.cli bench --preset medium --seq 2048 --micro-batch 4 --ac selective
    torchrun --nproc_per_node=8 -m forgeminds_b200.cli.bench --dp-shard 8 --json out.json

Reports tokens/s, step latency (p50/p90), MFU (``--peak-tflops``), peak memory, host syncs per step
(``--syncs``) and can record a ``torch.profiler`` trace (``--profile DIR``). Steps are timed with
CUDA events on the GPU (host clock on CPU). Flags follow the reference's
``forgemind/cli/bench.py:22-64``.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch

PRESETS = {
    "tiny": dict(dim=256, n_layers=4, n_heads=8, n_kv_heads=4),
    "small": dict(dim=768, n_layers=12, n_heads=12, n_kv_heads=4),
    "medium": dict(dim=1024, n_layers=24, n_heads=16, n_kv_heads=4),
}


def parse(argv=None):
    p = argparse.ArgumentParser(prog="forgeminds-b200-bench", description="benchmark a training step")
    g = p.add_argument_group("model")
    g.add_argument("--preset", default="small", choices=sorted(PRESETS))
    g.add_argument("--seq", type=int, default=512)
    g.add_argument("--micro-batch", type=int, default=4)
    g.add_argument("--grad-accum", type=int, default=1)
    g.add_argument("--ffn-hidden", type=int, default=0)
    g.add_argument("--moe", action="store_true")
    g.add_argument("--experts", type=int, default=8)
    g.add_argument("--top-k", type=int, default=2)
    g.add_argument("--capacity-factor", type=float, default=0.0)
    g = p.add_argument_group("quantization")
    g.add_argument("--quant", default="none", choices=["none", "fp8", "int8", "int8_wo"])
    g.add_argument("--qbackend", default="auto", choices=["auto", "native", "te", "torchao"])
    g.add_argument("--optimizer-8bit", action="store_true")
    g = p.add_argument_group("parallelism")
    g.add_argument("--dp-replicate", type=int, default=1)
    g.add_argument("--dp-shard", type=int, default=1)
    g.add_argument("--tp", type=int, default=1)
    g.add_argument("--pp", type=int, default=1)
    g.add_argument("--ep", type=int, default=1)
    g.add_argument("--backend", default="native", choices=["native", "deepspeed"])
    g.add_argument("--zero", type=int, default=2)
    g = p.add_argument_group("offload / memory")
    g.add_argument("--offload-opt", action="store_true")
    g.add_argument("--offload-act", action="store_true")
    g.add_argument("--offload-experts", action="store_true")
    g.add_argument("--ac", default="none", choices=["none", "full", "selective"])
    g = p.add_argument_group("run")
    g.add_argument("--warmup", type=int, default=5)
    g.add_argument("--steps", type=int, default=30)
    g.add_argument("--optimizer", default="adamw", choices=["adamw", "muon"])
    g.add_argument("--engine", default="auto", choices=["auto", "native", "library"])
    g.add_argument("--peak-tflops", type=float, default=0.0)
    g.add_argument("--json", default=None)
    g.add_argument("--profile", default=None, metavar="DIR")
    g.add_argument("--profile-top", type=int, default=15)
    g.add_argument("--compile", action="store_true")
    g.add_argument("--no-prefetch", action="store_true")
    g.add_argument("--syncs", action="store_true")
    return p.parse_args(argv)


def build_config(a):
    from .. import ForgeConfig
    cfg = ForgeConfig()
    cfg.parallel.__dict__.update(dp_replicate=a.dp_replicate, dp_shard=a.dp_shard, tp=a.tp, pp=a.pp, ep=a.ep,
                                 backend=a.backend, zero_stage=a.zero)
    cfg.quant.__dict__.update(mode=a.quant, backend=a.qbackend, optimizer_8bit=a.optimizer_8bit)
    cfg.offload.optimizer, cfg.offload.activations, cfg.offload.experts = a.offload_opt, a.offload_act, a.offload_experts
    cfg.train.__dict__.update(max_steps=a.warmup + a.steps, warmup_steps=0, log_every=10 ** 9, ac=a.ac, ckpt_every=0,
                              eval_every=0, resume=False, grad_clip=1.0, compile=a.compile,
                              prefetch=not a.no_prefetch, grad_accum=a.grad_accum, optimizer=a.optimizer,
                              native={"auto": None, "native": True, "library": False}[a.engine])
    return cfg


def _quantile(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(q * (len(xs) - 1))))]


def main(argv=None):
    from .. import GPT, GPTConfig, SyntheticLM, Trainer, cleanup, moe_kwargs
    from ..perf import DeviceTimer, count_host_syncs
    from ..quant import resolve_backend
    a = parse(argv)
    cfg = build_config(a)
    mc = GPTConfig(vocab_size=32000, max_seq=a.seq, n_experts=a.experts if a.moe else 0, top_k=a.top_k,
                   ffn_hidden=a.ffn_hidden or None, capacity_factor=a.capacity_factor, **PRESETS[a.preset])
    ds = SyntheticLM(mc.vocab_size, a.seq, n=max(256, a.micro_batch * a.grad_accum * (a.warmup + a.steps) * 2))
    tr = Trainer(lambda ctx: GPT(mc, moe_kwargs(ctx, cfg) if a.moe else None), cfg, ds, micro_batch=a.micro_batch,
                 peak_flops=a.peak_tflops * 1e12 or None)
    ctx = tr.ctx
    on_gpu = ctx.device.type == "cuda"
    if on_gpu:
        torch.cuda.reset_peak_memory_stats()
    resolved = resolve_backend(cfg.quant) if a.quant != "none" else "none"
    prof = None
    if a.profile:
        from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if on_gpu else [])
        prof = profile(activities=acts, record_shapes=True, profile_memory=True,
                       schedule=schedule(wait=0, warmup=1, active=3, repeat=1),
                       on_trace_ready=tensorboard_trace_handler(a.profile) if ctx.rank == 0 else None)
        prof.__enter__()
    timers, losses = [], []
    audit = counter = None
    for i in range(a.warmup + a.steps):
        if i == a.warmup and a.syncs:
            audit = count_host_syncs(capture_stack=False, count_cpu=not on_gpu)
            counter = audit.__enter__()
        t = DeviceTimer(ctx.device).start()
        m = tr.train_step()
        t.stop()
        if i >= a.warmup:
            timers.append(t)
            losses.append(m["loss"])
        if prof is not None:
            if on_gpu:
                torch.cuda.synchronize()
            prof.step()
    if audit is not None:
        audit.__exit__(None, None, None)
    if on_gpu:
        torch.cuda.synchronize()
    times = [t.elapsed_ms() / 1e3 for t in timers]
    if prof is not None:
        prof.__exit__(None, None, None)
        if ctx.rank == 0:
            key = "cuda_time_total" if on_gpu else "cpu_time_total"
            print(prof.key_averages().table(sort_by=key, row_limit=a.profile_top))
    tokens = a.micro_batch * a.seq * a.grad_accum * ctx.dp_world
    med = statistics.median(times)
    res = {
        "preset": a.preset, "seq": a.seq, "micro_batch": a.micro_batch, "grad_accum": a.grad_accum, "moe": a.moe,
        "world": ctx.world, "device": str(ctx.device),
        "gpu": torch.cuda.get_device_name(ctx.device) if on_gpu else "cpu",
        "engine": "native" if tr.store is not None else "library",
        "quant_mode": a.quant, "quant_requested": a.qbackend, "quant_resolved": resolved,
        "parallel": {"dp_replicate": a.dp_replicate, "dp_shard": a.dp_shard, "tp": a.tp, "pp": a.pp, "ep": a.ep},
        "offload": {"opt": a.offload_opt, "act": a.offload_act, "experts": a.offload_experts},
        "ac": a.ac, "backend": a.backend,
        "params_M": round(sum(p.numel() for p in tr.raw.parameters()) / 1e6, 2),
        "step_ms_p50": round(med * 1e3, 2), "step_ms_p90": round(_quantile(times, 0.9) * 1e3, 2),
        "tok_s": round(tokens / med, 1), "loss_last": round(losses[-1], 4),
        "timing": "cuda events" if on_gpu else "host clock",
    }
    if on_gpu:
        res["peak_mem_gb"] = round(torch.cuda.max_memory_allocated() / 2 ** 30, 2)
    if counter is not None:
        res["host_syncs_per_step"] = round(counter.own / max(1, a.steps), 2)
        res["host_syncs_torch_per_step"] = round(counter.external / max(1, a.steps), 2)
    if a.peak_tflops:
        res["mfu_pct"] = round(tr.raw.flops_per_token(a.seq) * res["tok_s"] / (a.peak_tflops * 1e12 * ctx.world) * 100, 2)
    tr.close()
    if ctx.rank == 0:
        print("\n=== forgeminds_b200 benchmark ===")
        for k, v in res.items():
            print(f"{k:>26}: {v}")
        if a.json:
            with open(a.json, "w") as f:
                json.dump(res, f, indent=2)
    cleanup()
    return res


if __name__ == "__main__":
    main()
