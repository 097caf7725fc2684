"""Per-kernel timings: eager PyTorch vs (optionally) ``torch.compile`` vs this library's kernels.

    python -m forgeminds_b200.cli kbench                         # every op, bf16, LLM-sized shapes
    python -m forgeminds_b200.cli kbench --ops rms_norm,gemm      # a subset
    python -m forgeminds_b200.cli kbench --mode fwd               # forward only
    python -m forgeminds_b200.cli kbench --check --tolerance 0.05 # exit 3 if a kernel loses to the best baseline
    python -m forgeminds_b200.cli kbench --json kernels.json

Each figure is the minimum over ``--iters`` runs timed with CUDA events after warm-up, with an L2
flush (a 256 MB write) before every timed run; the table also gives the achieved fraction of the
measured HBM bandwidth or bf16 GEMM peak (``MEASURED_PEAKS.json`` when present). On a machine
without a GPU every column runs the same PyTorch expression, so ``--check`` refuses to run there
(exit 2) unless ``--allow-cpu`` is given. Flags follow the reference's ``forgemind/cli/kbench.py:174-204``.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import time

import torch
import torch.nn.functional as F

DEFAULT_OPS = ["rms_norm", "add_rms_norm", "swiglu", "swiglu_split", "qk_norm_rope", "kl_div_logits",
               "newton_schulz", "topk", "softmax", "gemm", "attention", "cross_entropy"]


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def _sum(out):
    if isinstance(out, (tuple, list)):
        return sum(o.float().sum() for o in out if torch.is_tensor(o) and o.is_floating_point())
    return out.float().sum()


def build_case(op, a, device, dtype):
    """Returns ``(inputs, eager_fn, kernel_fn, bytes_moved, flops, differentiable)``."""
    from .. import kernels as K
    from ..kernels import reference as R
    tok, dim, hid = a.tokens, a.dim, a.hidden
    r = lambda *s: torch.randn(*s, device=device, dtype=dtype)          # noqa: E731
    es = torch.finfo(dtype).bits // 8
    if op == "rms_norm":
        x, w = r(tok, dim).requires_grad_(), torch.ones(dim, device=device, requires_grad=True)
        return (x, w), lambda: F.rms_norm(x, (dim,), w.to(dtype), 1e-6), lambda: K.rms_norm(x, w, 1e-6), 2 * tok * dim * es, 0, True
    if op == "add_rms_norm":
        x, d, w = r(tok, dim).requires_grad_(), r(tok, dim).requires_grad_(), torch.ones(dim, device=device, requires_grad=True)
        return (x, d, w), lambda: R.add_rms_norm(x, d, w.to(dtype), 1e-6), lambda: K.add_rms_norm(x, d, w, 1e-6), 4 * tok * dim * es, 0, True
    if op == "swiglu":
        g, u = r(tok, hid).requires_grad_(), r(tok, hid).requires_grad_()
        return (g, u), lambda: F.silu(g) * u, lambda: K.swiglu(g, u), 3 * tok * hid * es, 0, True
    if op == "swiglu_split":
        x = r(tok, 2 * hid).requires_grad_()
        return (x,), lambda: F.silu(x[..., :hid]) * x[..., hid:], lambda: K.swiglu_split(x), 3 * tok * hid * es, 0, True
    if op == "qk_norm_rope":
        B, T, H, D = a.batch, a.seq, a.heads, a.head_dim
        x, w = r(B, T, H, D).requires_grad_(), torch.ones(D, device=device, requires_grad=True)
        inv = 10000.0 ** (-torch.arange(0, D, 2, device=device, dtype=torch.float32) / D)
        ang = torch.outer(torch.arange(T, device=device, dtype=torch.float32), inv)
        cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
        return (x, w), lambda: R.qk_norm_rope(x, w, cos, sin), lambda: K.qk_norm_rope(x, w, cos, sin), 2 * x.numel() * es, 0, True
    if op == "kl_div_logits":
        s, t = r(min(tok, 4096), a.vocab).requires_grad_(), r(min(tok, 4096), a.vocab)
        return (s,), lambda: R.kl_div_logits(s, t)[0], lambda: K.kl_div_logits(s, t), 3 * s.numel() * es, 0, True
    if op == "newton_schulz":
        g = r(4, 1024, 1024)
        fl = 4 * 5 * 3 * 2 * 1024 ** 3
        return (), lambda: R.newton_schulz(g, 5), lambda: K.newton_schulz(g, 5), 0, fl, False
    if op == "topk":
        x = r(512, a.vocab)
        return (), lambda: torch.topk(x, 64, dim=-1), lambda: K.topk(x, 64), x.numel() * es, 0, False
    if op == "softmax":
        x = r(tok, 128).requires_grad_()
        return (x,), lambda: torch.softmax(x, -1), lambda: K.softmax(x), 2 * x.numel() * es, 0, True
    if op == "gemm":
        x, w = r(tok, dim).requires_grad_(), (torch.randn(hid, dim, device=device) * 0.02).to(dtype).requires_grad_()
        from ..ops.functional import linear
        fl = 2 * tok * dim * hid
        kern = (lambda: linear(x, w)) if device.type == "cuda" else (lambda: F.linear(x, w))
        return (x, w), lambda: F.linear(x, w), kern, 0, fl, True
    if op == "attention":
        B, T, H, D = a.batch, a.seq, a.heads, a.head_dim
        Hkv = max(1, H // 4)
        qkv = r(B, T, (H + 2 * Hkv) * D).requires_grad_()

        def eager():
            q = qkv[..., :H * D].unflatten(-1, (H, D)).transpose(1, 2)
            k = qkv[..., H * D:(H + Hkv) * D].unflatten(-1, (Hkv, D)).transpose(1, 2)
            v = qkv[..., (H + Hkv) * D:].unflatten(-1, (Hkv, D)).transpose(1, 2)
            return F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        from ..ops.functional import attention_qkv
        kern = (lambda: attention_qkv(qkv, H, Hkv, D, True)) if device.type == "cuda" else eager
        return (qkv,), eager, kern, 0, 2 * B * H * T * T * D, True
    if op == "cross_entropy":
        n = min(tok, 8192)
        h = r(n, dim).requires_grad_()
        w = (torch.randn(a.vocab, dim, device=device) * 0.02).to(dtype).requires_grad_()
        y = torch.randint(0, a.vocab, (n,), device=device)
        from ..loss import chunked_cross_entropy, fused_linear_cross_entropy
        return (h, w), lambda: chunked_cross_entropy(h, w, y), lambda: fused_linear_cross_entropy(h, w, y), 0, 2 * n * dim * a.vocab, True
    raise ValueError(f"unknown op {op!r}")


def time_op(fn, inputs, mode, iters, warmup, device, flush):
    def once():
        out = fn()
        if mode != "fwd" and inputs:
            _sum(out).backward()
            for t in inputs:
                t.grad = None
    for _ in range(warmup):
        once()
    best = math.inf
    for _ in range(iters):
        if device.type == "cuda":
            if flush is not None:
                flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            once()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        else:
            t0 = time.perf_counter()
            once()
            best = min(best, (time.perf_counter() - t0) * 1e3)
    return best


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="forgeminds-b200-kbench")
    p.add_argument("--ops", default=",".join(DEFAULT_OPS))
    p.add_argument("--mode", default="fwd+bwd", choices=["fwd", "fwd+bwd"])
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    p.add_argument("--tokens", type=int, default=8192)
    p.add_argument("--dim", type=int, default=4096)
    p.add_argument("--hidden", type=int, default=11008)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--seq", type=int, default=2048)
    p.add_argument("--heads", type=int, default=32)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--vocab", type=int, default=32000)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--compile", action="store_true", help="also time torch.compile of the eager expression")
    p.add_argument("--check", action="store_true")
    p.add_argument("--tolerance", type=float, default=0.0)
    p.add_argument("--allow-cpu", action="store_true")
    p.add_argument("--json", default=None)
    a = p.parse_args(argv)
    on_gpu = torch.cuda.is_available()
    if a.check and not on_gpu and not a.allow_cpu:
        print("kbench --check needs a GPU: on CPU every column runs the same PyTorch expression")
        return 2
    device = torch.device("cuda" if on_gpu else "cpu")
    dtype = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    if not on_gpu:
        a.tokens, a.dim, a.hidden, a.batch, a.seq, a.heads, a.vocab = 256, 256, 512, 1, 128, 4, 2048
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if on_gpu else None
    hbm, tflops, src = _peaks()
    rows, lost = [], []
    for op in [o for o in a.ops.split(",") if o]:
        inputs, eager, kern, nbytes, flops, diff = build_case(op, a, device, dtype)
        mode = a.mode if diff else "fwd"
        ins = inputs if mode != "fwd" else ()
        t_eager = time_op(eager, ins, mode, a.iters, a.warmup, device, flush)
        t_comp = float("nan")
        if a.compile and on_gpu:
            try:
                t_comp = time_op(torch.compile(eager), ins, mode, a.iters, a.warmup + 2, device, flush)
            except Exception:
                pass
        t_kern = time_op(kern, ins, mode, a.iters, a.warmup, device, flush)
        mult = 1.0 if mode == "fwd" else 3.0
        frac = ""
        if on_gpu and flops:
            frac = f"{mult * flops / (t_kern * 1e-3) / 1e12 / tflops:.2f} of {src} bf16 peak"
        elif on_gpu and nbytes:
            frac = f"{(mult if mode != 'fwd' else 1.0) * nbytes / (t_kern * 1e-3) / 1e9 / hbm:.2f} of {src} HBM"
        best_base = min(t for t in (t_eager, t_comp) if t == t)
        rows.append(dict(op=op, mode=mode, eager_ms=t_eager, compile_ms=t_comp, kernel_ms=t_kern,
                         speedup_vs_best=best_base / t_kern, roofline=frac))
        if t_kern > best_base * (1 + a.tolerance):
            lost.append(op)
    print(f"{'op':16s} {'mode':8s} {'eager ms':>10s} {'compile ms':>11s} {'kernel ms':>10s} {'vs best':>8s}  roofline")
    for r in rows:
        print(f"{r['op']:16s} {r['mode']:8s} {r['eager_ms']:10.3f} {r['compile_ms']:11.3f} {r['kernel_ms']:10.3f} "
              f"{r['speedup_vs_best']:7.2f}x  {r['roofline']}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"device": torch.cuda.get_device_name() if on_gpu else "cpu", "rows": rows}, f, indent=1)
    if a.check and lost:
        print("slower than the best baseline:", ", ".join(lost))
        return 3
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
