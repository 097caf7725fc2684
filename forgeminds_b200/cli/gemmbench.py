"""The linear-layer products of a GPT block against cuBLAS, one line per product.

    python -m forgeminds_b200.cli gemmbench --tokens 8192 --dim 1024 --hidden 2816 --heads 16 --kv-heads 4 \\
        --head-dim 64 --vocab 32000

For every projection (qkv, wo, gate|up, down, lm_head) the forward product ``y = x W^T``, the input
gradient ``dx = dy W`` and the weight gradient ``dW += dy^T x`` (fp32 accumulation into an existing
buffer, as the trainer does) are timed with CUDA events: median of ``--iters`` runs, a 256 MB write
between runs so that every run starts with a cold L2. ``cuBLAS`` is ``torch.matmul`` on the same
operands (bf16 output); ``ideal`` is FLOPs over the measured sustained bf16 GEMM rate.
"""
from __future__ import annotations

import argparse
import json
import os


def _sustained_tflops() -> float:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f).get("bf16_tflops_sustained", 1400.0))
    return 1400.0


def main(argv=None) -> int:
    import torch

    from ..ops import functional as Fn
    p = argparse.ArgumentParser(prog="forgeminds_b200.cli gemmbench")
    p.add_argument("--tokens", type=int, default=8192)
    p.add_argument("--dim", type=int, default=1024)
    p.add_argument("--hidden", type=int, default=2816)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--kv-heads", type=int, default=4)
    p.add_argument("--head-dim", type=int, default=64)
    p.add_argument("--vocab", type=int, default=32000)
    p.add_argument("--iters", type=int, default=15)
    p.add_argument("--json", default=None)
    p.add_argument("--quant", action="store_true", help="also time the int8 / fp8 products of the MLP projections")
    a = p.parse_args(argv)
    if not torch.cuda.is_available():
        print("gemmbench needs a GPU")
        return 1
    dev, M = "cuda", a.tokens
    flush = torch.empty(64 * 1024 * 1024, device=dev)
    peak = _sustained_tflops()

    def t(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2] * 1e3

    layers = [("qkv", (a.heads + 2 * a.kv_heads) * a.head_dim, a.dim), ("wo", a.dim, a.heads * a.head_dim),
              ("gate|up", 2 * a.hidden, a.dim), ("down", a.dim, a.hidden), ("lm_head", a.vocab, a.dim)]
    rows = []
    print(f"{'layer':<9}{'product':<8}{'M x N x K':<22}{'ours us':>9}{'cuBLAS us':>11}{'ideal us':>10}{'ours TFLOP/s':>14}")
    for name, N, K in layers:
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
        dy = torch.randn(M, N, device=dev).to(torch.bfloat16)
        y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        dx = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        dw = torch.zeros(N, K, device=dev, dtype=torch.float32)
        dwb = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        ideal = flops / (peak * 1e12) * 1e6
        for kind, ours, ref, shape in (
                ("fwd", lambda: Fn.gemm(x, w, out=y), lambda: torch.matmul(x, w.t(), out=y), f"{M} x {N} x {K}"),
                ("dgrad", lambda: Fn.gemm(dy, w, b_mn=True, out=dx), lambda: torch.matmul(dy, w, out=dx), f"{M} x {K} x {N}"),
                ("wgrad", lambda: Fn.gemm(dy, x, a_mn=True, b_mn=True, out=dw, c=dw, beta=1.0, allow_split=True),
                 lambda: torch.matmul(dy.t(), x, out=dwb), f"{N} x {K} x {M}")):
            to, tr = t(ours), t(ref)
            rows.append(dict(layer=name, product=kind, shape=shape, ours_us=round(to, 1), cublas_us=round(tr, 1),
                             ideal_us=round(ideal, 1), ours_tflops=round(flops / to / 1e6, 1)))
            print(f"{name:<9}{kind:<8}{shape:<22}{to:9.1f}{tr:11.1f}{ideal:10.1f}{flops / to / 1e6:14.1f}")
    tot_o, tot_r = sum(r["ours_us"] for r in rows), sum(r["cublas_us"] for r in rows)
    print(f"sum: ours {tot_o:.1f} us, cuBLAS {tot_r:.1f} us ({tot_r / tot_o:.2f}x)")
    qrows = _quant_table(a, t) if a.quant else []
    if a.json:
        with open(a.json, "w") as f:
            json.dump(dict(rows=rows, quant=qrows, peak_tflops=peak), f, indent=2)
    return 0


def _quant_table(a, t):
    """8-bit forward products ``x W^T`` of the two MLP projections: this library's int8 (row scales) and
    fp8 (e4m3; 1x128 activation / 128x128 weight scales, or row scales) kernels with and without the
    activation quantiser, against the bf16 kernel and ``torch._int_mm`` / ``torch._scaled_mm``."""
    import torch

    from .. import ops
    from ..ops import functional as Fn
    C = ops.require()
    dev, M = "cuda", a.tokens
    st = ops.status_word(torch.device(dev))
    out = []
    print()
    print(f"{'M x N x K':<22}{'kind':<26}{'us':>9}{'TOP/s':>9}")
    for N, K in ((2 * a.hidden, a.dim), (a.dim, a.hidden)):
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
        y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        xi, xis = C.quant_rows(x, 0, 0)
        wi, wis = C.quant_rows(w, 0, 0)
        xf, xfs = C.quant_rows(x, 1, 128)
        wf, wfs = C.quant_tiles_fp8(w)
        xr, xrs = C.quant_rows(x, 1, 0)
        wr, wrs = C.quant_rows(w, 1, 0)
        cases = [("bf16 (this library)", lambda: Fn.gemm(x, w, out=y)),
                 ("int8 product", lambda: C.gemm8(xi, wi, xis, wis, 0, False, st)),
                 ("int8 quantise + product", lambda: _qmm(C, x, 0, 0, wi, wis, st)),
                 ("fp8 block-scaled product", lambda: C.gemm8(xf, wf, xfs, wfs, 1, False, st)),
                 ("fp8 block quantise + product", lambda: _qmm(C, x, 1, 128, wf, wfs, st)),
                 ("fp8 row-scaled product", lambda: C.gemm8(xr, wr, xrs, wrs, 1, False, st))]
        try:
            a8, b8 = xi.view(torch.int8), wi.view(torch.int8).t()
            torch._int_mm(a8, b8)
            cases.append(("torch._int_mm (no scales)", lambda: torch._int_mm(a8, b8)))
        except Exception as e:                                   # noqa: BLE001 - library support varies
            print(f"torch._int_mm unavailable: {type(e).__name__}")
        try:
            af, bf = xr.view(torch.float8_e4m3fn), wr.view(torch.float8_e4m3fn).t()
            sa, sb = xrs.view(M, 1).contiguous(), wrs.view(1, N).contiguous()
            torch._scaled_mm(af, bf, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
            cases.append(("torch._scaled_mm row scales", lambda: torch._scaled_mm(af, bf, scale_a=sa, scale_b=sb,
                                                                                  out_dtype=torch.bfloat16)))
        except Exception as e:                                   # noqa: BLE001
            print(f"torch._scaled_mm unavailable: {type(e).__name__}")
        for kind, fn in cases:
            us = t(fn)
            out.append(dict(shape=f"{M} x {N} x {K}", kind=kind, us=round(us, 1), tops=round(flops / us / 1e6, 1)))
            print(f"{M} x {N} x {K:<10}{kind:<26}{us:9.1f}{flops / us / 1e6:9.1f}")
    return out


def _qmm(C, x, kind, block, wq, ws, st):
    q, s = C.quant_rows(x, kind, block)
    return C.gemm8(q, wq, s, ws, kind, False, st)


if __name__ == "__main__":
    raise SystemExit(main())
