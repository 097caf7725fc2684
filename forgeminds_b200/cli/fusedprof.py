"""Single-rank forms of the fused compute + collective kernels, sized for a profiler capture.

    python -m forgeminds_b200.cli fusedprof --op rs_reduce
    ncu --set full --clock-control none -k regex:rs_reduce_kernel -s 2 -c 1 -o prof \\
        python -m forgeminds_b200.cli fusedprof --op rs_reduce

A profiler replays each captured kernel many times, which kernels that wait for other ranks cannot
survive, so a multi-rank job is never profiled. With a group of one rank the same kernels run with peer
tables of length one: every load and store that would cross NVLink goes to local memory instead, and
the counters show the kernel's own work (memory traffic, tensor-pipe activity, stalls). Cross-GPU
timings of the same kernels come from ``cli commbench`` (CUDA events, max over ranks).

Operands are larger than the 126 MB L2 but at most a few hundred MB, so a capture with ``--set full``
ends by itself within a minute or two. Each op prints its device time (CUDA events, median of 3 after 2
warm-up runs).
"""
from __future__ import annotations

import argparse
import statistics

import torch

OPS = ("rs_reduce", "adamw_push", "push_cast", "ag_gemm", "gemm_rs", "ep_layer")


def _timed(fn, warmup=2, iters=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return statistics.median(out)


def main(argv=None) -> int:
    from .. import ops
    from ..parallel.symm import SymmGroup
    ap = argparse.ArgumentParser(prog="forgeminds_b200.cli fusedprof")
    ap.add_argument("--op", default="all", choices=OPS + ("all",))
    ap.add_argument("--bucket-mb", type=int, default=256)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    a = ap.parse_args(argv)
    C = ops.require()
    dev = torch.device("cuda")
    sg = SymmGroup(None, dev, timeout_ms=5000, solo=True)
    slot = sg.reserve_slots(8)
    todo = OPS if a.op == "all" else (a.op,)
    n = a.bucket_mb * (1 << 20) // 4
    report = {}

    if "rs_reduce" in todo:
        grads = sg.alloc(n, torch.float32)
        grads.local.normal_()
        partial = torch.zeros(296, dtype=torch.float32, device=dev)

        def run():       # scale != 1 so that the reduced values are written back, as with several ranks
            C.comm_rs_reduce(grads.ptrs, 0, n, 0.5, partial, sg.flags.ptrs, slot, sg.next_epoch(slot), 0, sg.timeout_ms,
                             sg.status)
        report["rs_reduce"] = (_timed(run), f"{a.bucket_mb} MB fp32 bucket read, scaled, written, summed in squares")

    if "adamw_push" in todo or "push_cast" in todo:
        master = torch.randn(n, device=dev)
        grad = torch.randn(n, device=dev)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        shadow = sg.alloc(n, torch.bfloat16)
        chunk = int(C.comm_adam_chunk())
        offs = torch.arange(0, n, chunk, dtype=torch.int64, device=dev)
        lens = torch.full_like(offs, chunk, dtype=torch.int32)
        wds = torch.full((offs.numel(),), 0.1, dtype=torch.float32, device=dev)
        ctl = torch.tensor([1.0, 1.0], device=dev)
        if "adamw_push" in todo:
            report["adamw_push"] = (_timed(lambda: C.comm_adamw_push(master, grad, m, v, shadow.ptrs, offs, offs, lens, wds,
                                                                     1e-4, 0.9, 0.95, 1e-8, 0.1, 0.05, ctl)),
                                    f"AdamW on {a.bucket_mb} MB of fp32 masters, bf16 result stored once")
        if "push_cast" in todo:
            report["push_cast"] = (_timed(lambda: C.comm_push_cast(master, shadow.ptrs, offs, lens)),
                                   f"{a.bucket_mb} MB of fp32 masters rounded to bf16 and stored once")

    M, K = a.tokens, a.dim
    if "ag_gemm" in todo:
        n_col = 2 * a.hidden
        x_buf = sg.alloc(M * K, torch.bfloat16)
        x_buf.local.normal_()
        ready = torch.zeros(M // 128, dtype=torch.int32, device=dev)
        w_col = (torch.randn(n_col, K, device=dev) * 0.02).to(torch.bfloat16)
        y = torch.empty(M, n_col, dtype=torch.bfloat16, device=dev)

        def run():
            epoch = sg.next_epoch(slot + 1)
            C.comm_signal(sg.flags.ptrs, slot + 1, epoch, 0, sg.status)
            C.gemm_peer(x_buf.local.view(M, K), w_col, y, False, False, 1.0, False, 0, 1, 1, x_buf.ptrs, ready, [],
                        sg.flags.local, slot + 1, epoch, sg.timeout_ms, sg.status)
        report["ag_gemm"] = (_timed(run), f"gathered-operand instantiation, [{M} x {K}] @ [{K} x {n_col}], all rows local")

    if "gemm_rs" in todo:
        h_loc = torch.randn(M, a.hidden, device=dev).to(torch.bfloat16)
        w_row = (torch.randn(K, a.hidden, device=dev) * 0.02).to(torch.bfloat16)
        staging = sg.alloc(M * K, torch.bfloat16)
        red = torch.empty(M, K, dtype=torch.bfloat16, device=dev)

        def run():
            C.gemm_peer(h_loc, w_row, staging.local.view(M, K), False, False, 1.0, False, 0, 1, 0, [], None, staging.ptrs,
                        sg.flags.local, -1, 0, sg.timeout_ms, sg.status)
            C.comm_sum_partials(staging.local, None, red, 1)
        report["gemm_rs"] = (_timed(run), f"scattered-output instantiation, [{M} x {a.hidden}] @ [{a.hidden} x {K}] into "
                                          "the staging buffer, then the slice sum")

    if "ep_layer" in todo:
        from ..moe import MoE
        from ..parallel.ep import EPEngine
        torch.manual_seed(0)
        layer = MoE(1024, 2816, 8, 2, grouped_mm=True).to(dev)
        layer.ep_size, layer.ep_rank = 1, 0
        eng = EPEngine.__new__(EPEngine)
        eng.sg = sg
        eng.rank, eng.world = 0, 1
        eng.s_pub, eng.s_ys, eng.s_gpub, eng.s_dxs, eng.s_done = (sg.reserve_slots(1) for _ in range(5))
        eng._key = None
        x = (torch.randn(16384, 1024, device=dev) * 0.5).to(torch.bfloat16).requires_grad_()

        def run():
            out = eng.forward(layer, x)
            out.float().sum().backward()
        report["ep_layer"] = (_timed(run), "expert-parallel MoE layer (8 experts, top-2, 16384 tokens x 1024), dispatch / "
                                           "combine kernels with a group of one, forward + backward")

    torch.cuda.synchronize()
    sg.check()
    for name, (ms, what) in report.items():
        print(f"{name:<12}{ms:>9.3f} ms   {what}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
