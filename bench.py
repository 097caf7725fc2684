#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s, MFU) of the dense GPT of the baseline config
(dim 1024, 24 layers, 16 heads / 4 kv heads, SwiGLU 2816, seq 2048; micro-batch 4 x grad-accum 4 per
GPU, AdamW 3e-4, bf16, sharded data parallel over N GPUs, selective activation checkpointing).
``--config moe | llama8b | gpt2p7b`` run the other multi-GPU configurations of the baseline list
(expert parallel MoE; tp 2 x pp 2 x dp_shard; hybrid sharding 2 x N/2) through the same harness.

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
MOE = dict(n_experts=8, top_k=2, aux_coef=0.01)

# The benchmark configurations. "dense" is the headline (dense GPT, sharded data parallel); the others are
# the remaining multi-GPU configurations of the baseline list. `mesh(world)` gives the parallel layout,
# `ffn_mult` is how the reference reaches the same MLP width (it has no explicit width field).
CONFIGS = {
    "dense": dict(
        model=dict(vocab_size=32000, dim=1024, n_layers=24, n_heads=16, n_kv_heads=4, max_seq=2048),
        hidden=2816, ffn_mult=2.75, micro_batch=4, grad_accum=4, seq=2048,
        mesh=lambda w: dict(dp_shard=w), label=lambda w: f"dp_shard{w}",
        name="gpt dim1024 L24 h16/kv4 swiglu2816 vocab32000"),
    "moe": dict(
        model=dict(vocab_size=32000, dim=1024, n_layers=24, n_heads=16, n_kv_heads=4, max_seq=2048),
        hidden=2816, ffn_mult=2.75, micro_batch=4, grad_accum=4, seq=2048,
        mesh=lambda w: dict(dp_replicate=w, ep=w), label=lambda w: f"ep{w}+dp_replicate{w}",
        name="gpt dim1024 L24 h16/kv4 swiglu2816 vocab32000 moe8top2"),
    "llama8b": dict(
        model=dict(vocab_size=32000, dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, max_seq=4096,
                   rope_theta=500000.0),
        hidden=14336, ffn_mult=3.5, micro_batch=8, grad_accum=1, seq=4096, min_world=4,
        mesh=lambda w: dict(tp=2, pp=2, dp_shard=w // 4, pp_microbatches=8, pp_schedule="1f1b"),
        label=lambda w: f"tp2 x pp2(1f1b, 8 microbatches of 1) x dp_shard{w // 4}",
        name="llama-style 8B dim4096 L32 h32/kv8 swiglu14336 vocab32000 theta5e5"),
    "gpt2p7b": dict(
        model=dict(vocab_size=32000, dim=2560, n_layers=32, n_heads=32, n_kv_heads=8, max_seq=2048),
        hidden=6912, ffn_mult=2.7, micro_batch=2, grad_accum=1, seq=2048, min_world=2,
        mesh=lambda w: dict(dp_replicate=2, dp_shard=w // 2), label=lambda w: f"hsdp dp_replicate2 x dp_shard{w // 2}",
        name="gpt 2.7B dim2560 L32 h32/kv8(hd80) swiglu6912 vocab32000"),
}


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

    def __init__(self, vocab, device, micro_batch, seq, n=16, seed=1):
        g = torch.Generator(device=device).manual_seed(seed)
        self.pool = [torch.randint(0, vocab, (micro_batch, seq + 1), device=device, generator=g) for _ in range(n)]
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
def _train_fields(spec, args):
    return dict(max_steps=10 ** 6, grad_accum=spec["grad_accum"], lr=3e-4, bf16=True, ac="selective", resume=False,
                ckpt_every=0, log_every=10 ** 9, warmup_steps=100, seed=1234)


def _on_device(ctx, build):
    """Build the model directly on the GPU: an 8 B-parameter model in fp32 on the host, once per rank,
    would need 8 x 32 GB of host memory."""
    if ctx.device.type == "cuda":
        with torch.device(ctx.device):
            return build()
    return build()


def build_ours(args, world):
    sys.path.insert(0, ROOT)
    import forgeminds_b200 as fm
    spec = CONFIGS[args.config]
    cfg = fm.ForgeConfig()
    cfg.parallel.__dict__.update(spec["mesh"](world))
    cfg.train.__dict__.update(_train_fields(spec, args))
    if args.quant != "none":
        cfg.quant.mode = args.quant
    if args.optimizer != "adamw":
        cfg.train.optimizer = args.optimizer
    if args.offload_activations:
        cfg.offload.activations = True
    cfg.parallel.ep_slot_factor = args.ep_slot_factor
    # the MoE arm runs dropless, like the reference, which has no capacity factor: both arms do the same work
    extra = dict(MOE, capacity_factor=args.capacity_factor, z_coef=0.0) if args.config == "moe" else {}
    mc = fm.GPTConfig(ffn_hidden=spec["hidden"], **spec["model"], **extra)
    ds = Tokens(spec["model"]["vocab_size"], spec["seq"], n=max(256, spec["micro_batch"] * spec["grad_accum"] * world * 8))

    def make(ctx):
        return _on_device(ctx, lambda: fm.GPT(mc, fm.moe_kwargs(ctx, cfg) if args.config == "moe" else None))
    trainer = fm.Trainer(make, cfg, ds, micro_batch=spec["micro_batch"], peak_flops=None)
    return trainer, fm


def build_reference(args, world):
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "forgemind")):
        return None, "baseline/_ref/forgemind is missing (reference not installed)"
    sys.path.insert(0, ref)
    import forgemind as fm
    spec = CONFIGS[args.config]
    cfg = fm.ForgeConfig()
    cfg.parallel.__dict__.update(spec["mesh"](world))
    cfg.train.__dict__.update(_train_fields(spec, args))
    if args.offload_activations:
        cfg.offload.activations = True
    extra = dict(MOE, z_coef=0.0) if args.config == "moe" else {}
    mc = fm.GPTConfig(ffn_mult=spec["ffn_mult"], **spec["model"], **extra)
    assert ((int(mc.dim * mc.ffn_mult) + 63) // 64) * 64 == spec["hidden"]
    ds = Tokens(spec["model"]["vocab_size"], spec["seq"], n=max(256, spec["micro_batch"] * spec["grad_accum"] * world * 8))

    def make(ctx):
        build = lambda: fm.GPT(mc, fm.moe_kwargs(ctx, cfg) if args.config == "moe" else None)   # noqa: E731
        # the reference builds on the host and moves the model (its expert re-initialisation draws from a host
        # generator); only the multi-billion-parameter configurations are built on the GPU, for host memory
        return _on_device(ctx, build) if args.config in ("llama8b", "gpt2p7b") else build()
    trainer = fm.Trainer(make, cfg, ds, micro_batch=spec["micro_batch"])
    return trainer, fm


def reference_failed(rank, exc):
    """The unmodified reference raised on its own stock path (for example its fused AdamW over a mix of plain
    and distributed tensors when a tensor-parallel mesh has no sharded data-parallel axis): say so in the
    contract's ``unavailable`` form and leave without waiting for the other ranks' teardown."""
    if rank == 0:
        why = f"the reference raised {type(exc).__name__}: {str(exc).splitlines()[0][:300] if str(exc) else ''}"
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    sys.stdout.flush()
    os._exit(0)


TINY = dict(model=dict(vocab_size=32000, dim=256, n_layers=4, n_heads=8, n_kv_heads=2, max_seq=256, tie_embeddings=True),
            hidden=704, micro_batch=4, grad_accum=2, seq=256,
            name="tiny gpt dim256 L4 h8/kv2 swiglu704 vocab32000 tied (the reference's own width: ceil64(256 * 8 / 3))")


def run_tiny_cpu(args, world: int, rank: int) -> int:
    """The CPU configuration of the baseline list: tiny GPT, fp32, Gloo, data parallel over ``world`` processes
    (``torchrun --nproc-per-node 2 bench.py --config tiny [--impl reference]``). Both arms go through their public
    ``Trainer``; wall-clock time around exactly ``--steps`` steps between barriers, maximum over ranks. A plumbing
    number of this host's cores, not a B200 number: the line says ``"device": "cpu"``."""
    if args.impl == "reference":
        ref = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref, "forgemind")):
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/forgemind is missing"}))
            return 0
        sys.path.insert(0, ref)
        import forgemind as fm
        mc = fm.GPTConfig(**TINY["model"])
        assert ((int(mc.dim * mc.ffn_mult) + 63) // 64) * 64 == TINY["hidden"]
    else:
        sys.path.insert(0, ROOT)
        import forgeminds_b200 as fm
        mc = fm.GPTConfig(ffn_hidden=TINY["hidden"], **TINY["model"])
    cfg = fm.ForgeConfig()
    cfg.parallel.dp_replicate = world
    cfg.train.__dict__.update(max_steps=10 ** 6, grad_accum=TINY["grad_accum"], lr=3e-4, bf16=False, ac="none",
                              resume=False, ckpt_every=0, log_every=10 ** 9, warmup_steps=100, seed=1234)
    ds = Tokens(TINY["model"]["vocab_size"], TINY["seq"], n=256)
    trainer = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, ds, micro_batch=TINY["micro_batch"])
    assert trainer.ctx.device.type == "cpu"
    for _ in range(args.warmup):
        trainer.train_step()
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        loss = trainer.train_step()["loss"]
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    ms = max_over_ranks(ms, "cpu")
    trainer.close()
    tokens = TINY["micro_batch"] * TINY["seq"] * TINY["grad_accum"] * world
    if rank == 0:
        print(json.dumps({
            "metric": "tokens_per_sec", "value": tokens / (ms / 1e3), "unit": "tokens/s", "device": "cpu", "n_gpus": 0,
            "n_processes": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "impl": args.impl,
            "data": "synthetic uniform tokens, random-init weights", "final_loss": loss,
            "config": {"model": TINY["name"], "global_batch": TINY["micro_batch"] * TINY["grad_accum"] * world,
                       "micro_batch": TINY["micro_batch"], "grad_accum": TINY["grad_accum"], "seq_len": TINY["seq"],
                       "parallelism": f"dp_replicate{world} (gloo)", "optimizer": "adamw lr3e-4", "ac": "none",
                       "threads_per_process": torch.get_num_threads()}}), flush=True)
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    return 0


def full_model_flops_per_token(spec, moe: bool) -> int:
    """``6 * active parameters + 12 * layers * dim * seq`` of the WHOLE model (the reference's MFU
    convention, ``forgemind/models/gpt.py:239-246``), whatever slice of it this rank holds."""
    m = spec["model"]
    d, L, V, h = m["dim"], m["n_layers"], m["vocab_size"], spec["hidden"]
    hd = d // m["n_heads"]
    attn = d * (m["n_heads"] * hd) * 2 + d * (m["n_kv_heads"] * hd) * 2
    mlp = 3 * d * h
    if moe:
        mlp_active = MOE["top_k"] * mlp + MOE["n_experts"] * d         # routed experts + router
    else:
        mlp_active = mlp
    n_active = 2 * V * d + L * (attn + mlp_active + 2 * d) + d
    return 6 * n_active + 12 * L * d * spec["seq"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="dense", choices=sorted(CONFIGS) + ["tiny"],
                    help="tiny: the CPU / Gloo configuration (fp32), run under torchrun on this host's cores")
    ap.add_argument("--quant", default="none", choices=["none", "fp8", "int8"],
                    help="8-bit GEMMs of this library (the reference's fp8 / int8 need libraries the image lacks)")
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "muon"])
    ap.add_argument("--offload-activations", action="store_true")
    ap.add_argument("--capacity-factor", type=float, default=0.0,
                    help="MoE arm: 0 = dropless like the reference; 1.25 = the capacity the config names")
    ap.add_argument("--ep-slot-factor", type=float, default=0.0,
                    help="MoE arm of this library: dispatch buffers sized to this multiple of a rank's average share "
                         "of the routed rows (0 = the worst case; an overflow is raised, never dropped silently)")
    ap.add_argument("--no-exposed-comm", action="store_true", help="skip the extra timed phase with local-only comm")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        # single-process invocation asked for several GPUs: re-launch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29511"), __file__,
               *sys.argv[1:]]
        return subprocess.call(cmd)
    if args.config == "tiny":
        os.environ.setdefault("CUDA_VISIBLE_DEVICES", "")          # this configuration is a CPU run wherever it starts
        return run_tiny_cpu(args, world, rank)
    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device visible"}))
        return 0
    spec = CONFIGS[args.config]
    if world % spec.get("min_world", 1):
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": f"config {args.config} needs a multiple of "
                                                                f"{spec['min_world']} GPUs, got {world}"}))
        return 0
    args.warmup = max(3, args.warmup)

    if args.impl == "reference":
        try:
            trainer, fm = build_reference(args, world)
        except Exception as e:                      # noqa: BLE001 - any failure of the stock path is reported, not hidden
            reference_failed(rank, e)
        if trainer is None:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": fm}))
            return 0
    else:
        trainer, fm = build_ours(args, world)
    device = trainer.ctx.device
    dp_world = trainer.ctx.dp_world
    micro_batch, accum, seq = spec["micro_batch"], spec["grad_accum"], spec["seq"]
    flops_tok = full_model_flops_per_token(spec, args.config == "moe")
    if world == dp_world and trainer.ctx.pc.ep == 1:
        assert flops_tok == trainer.raw.flops_per_token(seq), (flops_tok, trainer.raw.flops_per_token(seq))
    tokens_per_step = micro_batch * seq * accum * dp_world
    pk = peaks()
    vocab = spec["model"]["vocab_size"]

    ours = args.impl == "ours"
    if ours:
        from forgeminds_b200 import ops

    # ---- device-timed: batches resident on the GPU
    host_feed = trainer.feed
    trainer.feed = DeviceFeed(vocab, device, micro_batch, seq)
    try:
        for _ in range(args.warmup):
            trainer.train_step()
    except Exception as e:                          # noqa: BLE001
        if args.impl != "reference":
            raise
        reference_failed(rank, e)
    launches0 = ops.require().launch_count() if ours else 0
    torch.cuda.reset_peak_memory_stats(device)
    with ClockSampler(device.index or 0) as clocks:
        ms = timed_steps(trainer.train_step, args.steps, device)
    launches = (ops.require().launch_count() - launches0) if ours else None
    clock_info = clocks.summary()

    # ---- end to end: pinned host batches copied every micro-batch, loss read back every step
    dev_feed = trainer.feed
    trainer.feed = host_feed
    for _ in range(2):
        trainer.train_step()
    ms_e2e = timed_steps(trainer.train_step, args.steps, device)
    loss = trainer.train_step()["loss"]
    peak_alloc = max_over_ranks(torch.cuda.max_memory_allocated(device) / 2 ** 30, device)
    free_b, total_b = torch.cuda.mem_get_info(device)
    in_use = max_over_ranks((total_b - free_b) / 2 ** 30, device)

    # ---- exposed communication: the same step with the data-parallel kernels reading and writing local memory
    # only (one-way switch, so it comes last); the difference to the real step is what the ranks wait for
    exposed = None
    if ours and world > 1 and not args.no_exposed_comm and getattr(trainer.eng, "detach_peers", lambda: False)():
        trainer.feed = dev_feed
        for _ in range(2):
            trainer.train_step()
        ms_local = timed_steps(trainer.train_step, args.steps, device)
        exposed = {"exposed_comm_ms": max(0.0, ms - ms_local), "ms_per_step_local_comm": ms_local,
                   "how": "same step with reduce-scatter / scalar exchange / weight push on this rank's memory only"}
    trainer.close()

    value = tokens_per_step / (ms / 1e3)
    e2e = tokens_per_step / (ms_e2e / 1e3)
    mfu = value * flops_tok / (pk["bf16_tflops_sustained"] * 1e12 * world)
    h2d = micro_batch * seq * 8 * 2 * accum          # int64 inputs + labels per rank and step
    dtype = "bf16" if args.quant == "none" or not ours else f"bf16 master weights, {args.quant} GEMMs"
    optim = "adamw lr3e-4" if args.optimizer == "adamw" or not ours else "muon (2-D block weights) + adamw lr3e-4"
    out = {
        "metric": "tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": dtype, "data": "synthetic uniform tokens, random-init weights",
        "impl": args.impl,
        "mfu_of_measured_sustained": mfu,
        "mfu_of_measured_burst": value * flops_tok / (pk["bf16_tflops"] * 1e12 * world),
        "config": {"model": spec["name"], "global_batch": micro_batch * accum * dp_world, "micro_batch": micro_batch,
                   "grad_accum": accum, "seq_len": seq, "parallelism": spec["label"](world),
                   "optimizer": optim, "ac": "selective",
                   "engine": (trainer.eng.name + ("+peer" if trainer.peer else "")) if ours else "reference Trainer",
                   "memory_layout": ("bf16 weights, fp32 gradients and the fp32 master buffer whole on every GPU (only the "
                                     "rank's own shard of the masters is updated between steps), optimizer moments "
                                     "sharded 1/dp_shard" if ours and getattr(trainer, "store", None) is not None
                                     else "as the wrapped torch.distributed strategy shards it"),
                   "l2": "per-step working set (weights+activations, >10 GB) exceeds the 126 MB L2"},
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 12 if dp_world == world else 16},
        "gpu_launches": launches,
        "clocks": clock_info,
        "final_loss": loss,
        "flops_per_token": flops_tok,
        "peak_mem_gb": peak_alloc,
        "device_mem_in_use_gb": in_use,
        "peaks": {k: pk.get(k) for k in ("bf16_tflops", "bf16_tflops_sustained", "hbm_gbs")},
    }
    if args.config == "moe":
        out["config"]["moe"] = "dropless" if not ours or args.capacity_factor <= 0 else f"capacity factor {args.capacity_factor}"
    if exposed is not None:
        out.update(exposed)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
