"""Timings of the peer-memory kernels against their NCCL formulations (run under torchrun, one rank per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m forgeminds_b200.cli commbench --json comm.json

Every figure is the median of ``--iters`` runs timed with CUDA events on the launching stream after
warm-up, with a NCCL barrier before each run, and the MAX over ranks. For each fused kernel the table
gives the roofline target ``max(FLOPs / measured bf16 GEMM rate, bytes over NVLink / 770 GB/s, bytes of
local HBM traffic / measured copy bandwidth)`` and the achieved fraction, next to the unfused NCCL formulation of the same step.

  rs_reduce     pull reduce-scatter of a gradient bucket (+ sum of squares)    vs  reduce_scatter_tensor
  adamw_push    sharded AdamW + bf16 store into every rank's weights           vs  fused AdamW on the shard + all_gather
  ag_gemm       all-gather -> GEMM (column-parallel projection)                vs  all_gather_into_tensor + GEMM
  gemm_rs       GEMM -> reduce-scatter (row-parallel projection) + slice sum    vs  GEMM + reduce_scatter_tensor
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0          # measured peer copy bandwidth per direction per GPU on this pool


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops", 1590.0)), float(d.get("hbm_gbs", 6650.0)), "measured"
    return 1590.0, 6650.0, "fallback"


def _time(fn, iters, warmup, device):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    out = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize(device)
        out.append(e0.elapsed_time(e1))
    t = torch.tensor([statistics.median(out)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None) -> int:
    from .. import ops
    from ..parallel.symm import SymmGroup
    p = argparse.ArgumentParser(prog="forgeminds_b200.cli commbench")
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--bucket-mb", type=int, default=256, help="gradient bucket size (fp32) for rs_reduce / adamw_push")
    p.add_argument("--tokens", type=int, default=8192)
    p.add_argument("--dim", type=int, default=4096)
    p.add_argument("--hidden", type=int, default=14336)
    p.add_argument("--json", default=None)
    a = p.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    C = ops.require()
    sg = SymmGroup(None, dev, timeout_ms=10000)
    tflops, hbm_gbs, src = _peaks()
    rows = []

    def add(name, fused_ms, nccl_ms, flops, link_bytes, note="", hbm_bytes=0.0):
        target = max(flops / (tflops * 1e12), link_bytes / (NVLINK_GBS * 1e9), hbm_bytes / (hbm_gbs * 1e9)) * 1e3
        rows.append(dict(op=name, fused_ms=round(fused_ms, 4), nccl_ms=round(nccl_ms, 4), target_ms=round(target, 4),
                         achieved=round(target / fused_ms, 3) if fused_ms > 0 else None, note=note))

    # ---------------------------------------------------------------- reduce-scatter of a gradient bucket
    n = a.bucket_mb * (1 << 20) // 4
    n -= n % (world * 4096)
    shard = n // world
    grads = sg.alloc(n, torch.float32)
    grads.local.normal_()
    partial = torch.zeros(296, dtype=torch.float32, device=dev)
    slot = sg.reserve_slots(8)

    def rs_fused():
        C.comm_rs_reduce(grads.ptrs, rank * shard, shard, 1.0 / world, partial, sg.flags.ptrs, slot, sg.next_epoch(slot),
                         rank, sg.timeout_ms, sg.status)
        sg.barrier(slot + 1)             # nobody overwrites its bucket while a peer still reads it

    out_shard = torch.empty(shard, dtype=torch.float32, device=dev)

    def rs_nccl():
        dist.reduce_scatter_tensor(out_shard, grads.local, op=dist.ReduceOp.AVG)
        out_shard.square().sum()

    add("rs_reduce", _time(rs_fused, a.iters, a.warmup, dev), _time(rs_nccl, a.iters, a.warmup, dev), 0.0,
        shard * 4 * (world - 1), f"{a.bucket_mb} MB fp32 bucket, {world} ranks", hbm_bytes=shard * 8.0)

    # ---------------------------------------------------------------- sharded AdamW + push
    master = torch.randn(n, device=dev)
    m = torch.zeros(shard, device=dev)
    v = torch.zeros(shard, device=dev)
    shadow = sg.alloc(n, torch.bfloat16)
    chunk = int(C.comm_adam_chunk())
    offs = torch.arange(rank * shard, (rank + 1) * shard, chunk, dtype=torch.int64, device=dev)
    soffs = offs - rank * shard
    lens = torch.full_like(offs, chunk, dtype=torch.int32)
    wds = torch.full((offs.numel(),), 0.1, dtype=torch.float32, device=dev)
    ctl = torch.tensor([1.0, 1.0], device=dev)

    def push_fused():
        C.comm_adamw_push(master, grads.local, m, v, shadow.ptrs, offs, soffs, lens, wds, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.05, ctl)
        sg.barrier(slot + 2)

    p_shard = torch.nn.Parameter(master[rank * shard:(rank + 1) * shard].clone())
    p_shard.grad = grads.local[rank * shard:(rank + 1) * shard].clone()
    opt = torch.optim.AdamW([p_shard], lr=1e-4, fused=True)
    full_bf16 = torch.empty(n, dtype=torch.bfloat16, device=dev)

    def push_nccl():
        opt.step()
        dist.all_gather_into_tensor(full_bf16, p_shard.detach().to(torch.bfloat16))

    add("adamw_push", _time(push_fused, a.iters, a.warmup, dev), _time(push_nccl, a.iters, a.warmup, dev), 0.0,
        shard * 2 * (world - 1), "fp32 master + moments on the shard, bf16 to every rank", hbm_bytes=shard * 30.0)

    # ---------------------------------------------------------------- all-gather -> GEMM
    M, K = a.tokens, a.dim
    ms = M // world
    n_col = 2 * a.hidden // world
    n_col -= n_col % 8
    x_buf = sg.alloc(M * K, torch.bfloat16)                  # gather buffer: own slice published, the rest pulled
    x_buf.local.normal_()
    ready = torch.zeros(M // 128, dtype=torch.int32, device=dev)
    w_col = torch.randn(n_col, K, device=dev).to(torch.bfloat16) * 0.02
    y = torch.empty(M, n_col, dtype=torch.bfloat16, device=dev)

    def ag_fused():
        epoch = sg.next_epoch(slot + 3)
        C.comm_signal(sg.flags.ptrs, slot + 3, epoch, rank, sg.status)
        C.gemm_peer(x_buf.local.view(M, K), w_col, y, False, False, 1.0, False, rank, world, 1, x_buf.ptrs, ready, [],
                    sg.flags.local, slot + 3, epoch, sg.timeout_ms, sg.status)
        sg.barrier(slot + 4)

    x_full = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    x_own = x_buf.local.view(M, K)[rank * ms:(rank + 1) * ms].clone()

    def ag_nccl():
        dist.all_gather_into_tensor(x_full, x_own)
        torch.matmul(x_full, w_col.t(), out=y)

    def local_only():
        C.gemm(x_full, w_col, y, None, False, False, 1.0, 0.0, None, False, sg.status, 0)

    add("ag_gemm", _time(ag_fused, a.iters, a.warmup, dev), _time(ag_nccl, a.iters, a.warmup, dev), 2.0 * M * n_col * K,
        ms * K * 2 * (world - 1), f"[{M} x {K}] rows gathered, {n_col} output columns per rank")
    rows[-1]["local_gemm_ms"] = round(_time(local_only, a.iters, a.warmup, dev), 4)

    # ---------------------------------------------------------------- GEMM -> reduce-scatter
    k_row = a.hidden // world
    k_row -= k_row % 8
    h_loc = torch.randn(M, k_row, device=dev).to(torch.bfloat16)
    w_row = torch.randn(K, k_row, device=dev).to(torch.bfloat16) * 0.02
    staging = sg.alloc(M * K, torch.bfloat16)                # [world, ms, K]
    red = torch.empty(ms, K, dtype=torch.bfloat16, device=dev)

    def rs_gemm_fused():
        C.gemm_peer(h_loc, w_row, staging.local.view(M, K), False, False, 1.0, False, rank, world, 0, [], None,
                    staging.ptrs, sg.flags.local, -1, 0, sg.timeout_ms, sg.status)
        sg.barrier(slot + 6)
        C.comm_sum_partials(staging.local, None, red, world)
        sg.barrier(slot + 5)                                  # nobody writes the next partials before this sum is done

    part = torch.empty(M, K, dtype=torch.bfloat16, device=dev)

    def rs_gemm_nccl():
        torch.matmul(h_loc, w_row.t(), out=part)
        dist.reduce_scatter_tensor(red, part)

    def local_rs():
        C.gemm(h_loc, w_row, part, None, False, False, 1.0, 0.0, None, False, sg.status, 0)

    add("gemm_rs", _time(rs_gemm_fused, a.iters, a.warmup, dev), _time(rs_gemm_nccl, a.iters, a.warmup, dev),
        2.0 * M * K * k_row, ms * K * 2 * (world - 1),
        f"[{M} x {k_row}] @ [{k_row} x {K}], bf16 partial tiles stored into the owners' staging buffers, then summed")
    rows[-1]["local_gemm_ms"] = round(_time(local_rs, a.iters, a.warmup, dev), 4)

    torch.cuda.synchronize(dev)
    sg.check()
    if rank == 0:
        print(f"peaks: {tflops:.0f} TFLOP/s bf16 ({src}), NVLink {NVLINK_GBS:.0f} GB/s per direction; {world} ranks")
        print(f"{'op':<12}{'fused ms':>10}{'NCCL ms':>10}{'target ms':>11}{'achieved':>10}  note")
        for r in rows:
            extra = f" (same product on local operands: {r['local_gemm_ms']:.3f} ms)" if "local_gemm_ms" in r else ""
            print(f"{r['op']:<12}{r['fused_ms']:>10.3f}{r['nccl_ms']:>10.3f}{r['target_ms']:>11.3f}{r['achieved']:>10.2f}  {r['note']}{extra}")
        if a.json:
            with open(a.json, "w") as f:
                json.dump(dict(world=world, rows=rows), f, indent=2)
    dist.barrier()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
