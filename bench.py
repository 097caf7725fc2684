#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s, MFU) of the dense GPT of the baseline config
(dim 1024, 24 layers, 16 heads / 4 kv heads, SwiGLU 2816, seq 2048; micro-batch 4 x grad-accum 4 per
GPU, AdamW 3e-4, bf16, sharded data parallel over N GPUs, selective activation checkpointing).

    python bench.py --gpus 1 --steps 5 --warmup 3                  # this library
    python bench.py --impl reference --gpus 1 --steps 5 --warmup 3 # unmodified reference (baseline/_ref)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3

Rank 0 prints one JSON line. ``value`` is the whole-job tokens/s timed on the device (CUDA events,
max over ranks) with token batches already resident on the GPU; ``e2e`` is the same loop through the
public ``Trainer`` API with every micro-batch copied from pinned host memory and the step's loss read
back, which is how a user runs it. Synthetic uniform tokens, random-initialised weights.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
MODEL = dict(vocab_size=32000, dim=1024, n_layers=24, n_heads=16, n_kv_heads=4, max_seq=2048)
HIDDEN = 2816
MICRO_BATCH, GRAD_ACCUM, SEQ = 4, 4, 2048
MOE = dict(n_experts=8, top_k=2, aux_coef=0.01)


# ------------------------------------------------------------------------------ helpers
class Tokens(torch.utils.data.Dataset):
    """Uniform random tokens from a fixed seed; labels are the inputs shifted left by one."""

    def __init__(self, vocab, seq, n, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.t = torch.randint(0, vocab, (n, seq + 1), generator=g)

    def __len__(self):
        return self.t.shape[0]

    def __getitem__(self, i):
        row = self.t[i]
        return {"input_ids": row[:-1], "labels": row[1:]}


class DeviceFeed:
    """Stands in for the trainer's batch stream with batches that already live on the GPU."""

    def __init__(self, vocab, device, n=16, seed=1):
        g = torch.Generator(device=device).manual_seed(seed)
        self.pool = [torch.randint(0, vocab, (MICRO_BATCH, SEQ + 1), device=device, generator=g) for _ in range(n)]
        self.i = 0
        self.epoch, self.batches = 0, 0

    def next(self):
        t = self.pool[self.i % len(self.pool)]
        self.i += 1
        return t[:, :-1], t[:, 1:]

    def close(self):
        pass

    def resume(self, *a):
        pass


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        return False

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def max_over_ranks(ms: float, device) -> float:
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def timed_steps(step_fn, steps: int, device) -> float:
    """Milliseconds per step: barrier + synchronize, CUDA events around exactly ``steps`` steps,
    synchronize + barrier, maximum over ranks."""
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step_fn()
    stop.record()
    torch.cuda.synchronize()
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
    return max_over_ranks(start.elapsed_time(stop) / steps, device)


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "fallback": True}


# ------------------------------------------------------------------------------ the two arms
def build_ours(args, world):
    sys.path.insert(0, ROOT)
    import forgeminds_b200 as fm
    cfg = fm.ForgeConfig()
    cfg.parallel.dp_shard = world if args.config != "moe" else 1
    cfg.parallel.dp_replicate = 1 if args.config != "moe" else world
    if args.config == "moe":
        cfg.parallel.ep = world
    cfg.train.__dict__.update(max_steps=10 ** 6, grad_accum=GRAD_ACCUM, lr=3e-4, bf16=True, ac="selective",
                              resume=False, ckpt_every=0, log_every=10 ** 9, warmup_steps=100, seed=1234)
    extra = dict(MOE, capacity_factor=1.25, z_coef=0.0) if args.config == "moe" else {}
    mc = fm.GPTConfig(ffn_hidden=HIDDEN, **MODEL, **extra)
    ds = Tokens(MODEL["vocab_size"], SEQ, n=max(256, MICRO_BATCH * GRAD_ACCUM * world * 8))

    def make(ctx):
        return fm.GPT(mc, fm.moe_kwargs(ctx, cfg) if args.config == "moe" else None)
    trainer = fm.Trainer(make, cfg, ds, micro_batch=MICRO_BATCH, peak_flops=None)
    return trainer, fm


def build_reference(args, world):
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "forgemind")):
        return None, "baseline/_ref/forgemind is missing (reference not installed)"
    sys.path.insert(0, ref)
    import forgemind as fm
    cfg = fm.ForgeConfig()
    if args.config == "moe":
        cfg.parallel.dp_replicate, cfg.parallel.ep = world, world
    else:
        cfg.parallel.dp_shard = world
    cfg.train.__dict__.update(max_steps=10 ** 6, grad_accum=GRAD_ACCUM, lr=3e-4, bf16=True, ac="selective",
                              resume=False, ckpt_every=0, log_every=10 ** 9, warmup_steps=100, seed=1234)
    extra = dict(MOE, z_coef=0.0) if args.config == "moe" else {}
    mc = fm.GPTConfig(ffn_mult=2.75, **MODEL, **extra)          # ceil64(1024 * 2.75) = 2816
    ds = Tokens(MODEL["vocab_size"], SEQ, n=max(256, MICRO_BATCH * GRAD_ACCUM * world * 8))

    def make(ctx):
        return fm.GPT(mc, fm.moe_kwargs(ctx, cfg) if args.config == "moe" else None)
    trainer = fm.Trainer(make, cfg, ds, micro_batch=MICRO_BATCH)
    return trainer, fm


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="dense", choices=["dense", "moe"])
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        # single-process invocation asked for several GPUs: re-launch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29511"), __file__,
               *sys.argv[1:]]
        return subprocess.call(cmd)
    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device visible"}))
        return 0
    args.warmup = max(3, args.warmup)

    if args.impl == "reference":
        trainer, fm = build_reference(args, world)
        if trainer is None:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": fm}))
            return 0
    else:
        trainer, fm = build_ours(args, world)
    device = trainer.ctx.device
    model = trainer.raw
    flops_tok = model.flops_per_token(SEQ)
    tokens_per_step = MICRO_BATCH * SEQ * GRAD_ACCUM * world
    pk = peaks()

    launches0 = 0
    if args.impl == "ours":
        from forgeminds_b200 import ops
        launches0 = ops.require().launch_count()

    # ---- device-timed: batches resident on the GPU
    host_feed = trainer.feed
    trainer.feed = DeviceFeed(MODEL["vocab_size"], device)
    for _ in range(args.warmup):
        trainer.train_step()
    if args.impl == "ours":
        launches0 = ops.require().launch_count()
    with ClockSampler(device.index or 0) as clocks:
        ms = timed_steps(trainer.train_step, args.steps, device)
    launches = (ops.require().launch_count() - launches0) if args.impl == "ours" else None
    clock_info = clocks.summary()

    # ---- end to end: pinned host batches copied every micro-batch, loss read back every step
    trainer.feed = host_feed
    for _ in range(2):
        trainer.train_step()
    ms_e2e = timed_steps(trainer.train_step, args.steps, device)
    loss = trainer.train_step()["loss"]
    trainer.close()

    value = tokens_per_step / (ms / 1e3)
    e2e = tokens_per_step / (ms_e2e / 1e3)
    mfu = value * flops_tok / (pk["bf16_tflops_sustained"] * 1e12 * world)
    h2d = MICRO_BATCH * SEQ * 8 * 2 * GRAD_ACCUM          # int64 inputs + labels per rank and step
    out = {
        "metric": "tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform tokens, random-init weights",
        "impl": args.impl,
        "mfu_of_measured_sustained": mfu,
        "mfu_of_measured_burst": value * flops_tok / (pk["bf16_tflops"] * 1e12 * world),
        "config": {"model": "gpt dim1024 L24 h16/kv4 swiglu2816 vocab32000" + (" moe8top2" if args.config == "moe" else ""),
                   "global_batch": MICRO_BATCH * GRAD_ACCUM * world, "micro_batch": MICRO_BATCH,
                   "grad_accum": GRAD_ACCUM, "seq_len": SEQ,
                   "parallelism": (f"ep{world}+dp_replicate{world}" if args.config == "moe" else f"dp_shard{world}"),
                   "optimizer": "adamw lr3e-4", "ac": "selective",
                   "l2": "per-step working set (weights+activations, >10 GB) exceeds the 126 MB L2"},
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 12},
        "gpu_launches": launches,
        "clocks": clock_info,
        "final_loss": loss,
        "flops_per_token": flops_tok,
        "peaks": {k: pk.get(k) for k in ("bf16_tflops", "bf16_tflops_sustained", "hbm_gbs")},
    }
    if rank == 0:
        print(json.dumps(out), flush=True)
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
