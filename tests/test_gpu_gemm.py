"""tcgen05 GEMM against an fp32 PyTorch reference: all operand layouts, epilogues, ragged edges."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


def _mk(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(rows, cols, device="cuda", generator=g) * 0.5).to(torch.bfloat16)


def _close(out, ref, K):
    tol = 2e-2 * (K ** 0.5) * 0.25 + 1e-2
    err = (out.float() - ref).abs().max().item()
    assert err < tol, f"max err {err} > {tol}"
    rel = (out.float() - ref).norm() / ref.norm().clamp(min=1e-6)
    assert rel < 1e-2, f"relative error {rel}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (512, 384, 320), (1024, 1536, 1024), (200, 136, 72)])
def test_layouts(M, N, K, a_mn, b_mn, cuda_status):
    from forgeminds_b200.ops.functional import gemm
    a = _mk(K, M, 1) if a_mn else _mk(M, K, 1)
    b = _mk(K, N, 2) if b_mn else _mk(N, K, 2)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    _close(out, _ref(a, b, a_mn, b_mn), K)


@pytest.mark.parametrize("bn", [128, 256])
def test_tile_widths(bn, cuda_status):
    from forgeminds_b200.ops.functional import gemm
    a, b = _mk(640, 512, 3), _mk(768, 512, 4)
    out = gemm(a, b, force_bn=bn)
    _close(out, _ref(a, b, False, False), 512)


def test_residual_epilogue(cuda_status):
    from forgeminds_b200.ops.functional import gemm
    a, b, r = _mk(512, 256, 5), _mk(384, 256, 6), _mk(512, 384, 7)
    out = gemm(a, b, c=r, beta=1.0)
    _close(out, _ref(a, b, False, False) + r.float(), 256)


def test_fp32_accumulate_and_split_k(cuda_status):
    from forgeminds_b200.ops.functional import gemm
    # weight-gradient shape: few output tiles, long reduction -> split-K with atomics
    dy, x = _mk(8192, 256, 8), _mk(8192, 384, 9)
    acc = torch.full((256, 384), 0.5, device="cuda")
    gemm(dy, x, a_mn=True, b_mn=True, out=acc, c=acc, beta=1.0, allow_split=True)
    ref = dy.float().t() @ x.float() + 0.5
    assert (acc - ref).abs().max() < 0.35
    assert (acc - ref).norm() / ref.norm() < 2e-3
    fresh = gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32, allow_split=True)
    assert (fresh - (ref - 0.5)).norm() / ref.norm() < 2e-3


def test_device_alpha(cuda_status):
    from forgeminds_b200.ops.functional import gemm
    a, b = _mk(256, 128, 10), _mk(256, 128, 11)
    s = torch.tensor([0.25], device="cuda")
    out = gemm(a, b, alpha=2.0, alpha_dev=s)
    _close(out, 0.5 * _ref(a, b, False, False), 128)


def test_strided_rows(cuda_status):
    from forgeminds_b200.ops.functional import gemm
    big = _mk(512, 1024, 12)
    a = big[:, 256:512]                       # row pitch 1024, 256 columns
    b = _mk(128, 256, 13)
    out = gemm(a, b)
    _close(out, a.float() @ b.float().t(), 256)


def test_linear_autograd(cuda_status):
    from forgeminds_b200.ops.functional import linear
    x = _mk(512, 256, 14).requires_grad_()
    w = torch.randn(384, 256, device="cuda", requires_grad=True) * 0.05
    w = w.detach().requires_grad_()
    res = _mk(512, 384, 15).requires_grad_()
    y = linear(x, w, res)
    g = _mk(512, 384, 16)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().to(torch.bfloat16).float().requires_grad_()
    rr = res.detach().float().requires_grad_()
    yr = xr @ wr.t() + rr
    yr.backward(g.float())
    assert (y.float() - yr).abs().max() < 0.1
    assert (x.grad.float() - xr.grad).norm() / xr.grad.norm() < 1e-2
    assert (w.grad - wr.grad).norm() / wr.grad.norm() < 1e-2
    assert torch.equal(res.grad, g)


def test_main_grad_accumulation(cuda_status):
    from forgeminds_b200.ops.functional import linear
    x = _mk(1024, 256, 17)
    w = (torch.randn(128, 256, device="cuda") * 0.05).requires_grad_()
    w._fm_main_grad = torch.zeros(128, 256, device="cuda")
    for _ in range(2):
        linear(x, w).sum().backward()
    assert w.grad is None
    ref = 2 * torch.ones(1024, 128, device="cuda").t() @ x.float()
    assert (w._fm_main_grad - ref).norm() / ref.norm() < 2e-3


def test_swiglu_fused_into_gemm_epilogues(cuda_status):
    """gate|up product with the activation from its epilogue; d(act) product with the SwiGLU backward in its epilogue."""
    from forgeminds_b200 import ops
    C = ops.require()
    torch.manual_seed(0)
    M, K, h, d = 384, 256, 640, 256
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w13 = (torch.randn(2 * h, K, device="cuda") * 0.1).to(torch.bfloat16)
    gu = torch.empty(M, 2 * h, dtype=torch.bfloat16, device="cuda")
    act = torch.empty(M, h, dtype=torch.bfloat16, device="cuda")
    C.gemm_swiglu_fwd(x, w13, gu, act, cuda_status)
    want_gu = (x.float() @ w13.float().T)
    assert (gu.float() - want_gu).abs().max() < 0.02 * want_gu.abs().max()
    g, u = gu[:, :h].float(), gu[:, h:].float()
    want_act = torch.nn.functional.silu(g) * u
    assert (act.float() - want_act).abs().max() < 0.02 * want_act.abs().max() + 1e-3
    # backward
    dy = (torch.randn(M, d, device="cuda") * 0.5).to(torch.bfloat16)
    w2 = (torch.randn(d, h, device="cuda") * 0.1).to(torch.bfloat16)
    dgu = torch.empty_like(gu)
    C.gemm_swiglu_bwd(dy, w2, gu, dgu, cuda_status)
    dact = (dy.float() @ w2.float()).to(torch.bfloat16).float()
    s = torch.sigmoid(g)
    want_dg = dact * u * s * (1 + g * (1 - s))
    want_du = dact * g * s
    assert (dgu[:, :h].float() - want_dg).abs().max() < 0.03 * want_dg.abs().max() + 1e-3
    assert (dgu[:, h:].float() - want_du).abs().max() < 0.03 * want_du.abs().max() + 1e-3


@pytest.mark.parametrize("seg,seq", [(64, 0), (64, 96), (128, 0), (32, 48)])
def test_row_dots_from_the_gemm_epilogue(seg, seq, cuda_status):
    from forgeminds_b200 import ops
    C = ops.require()
    torch.manual_seed(1)
    M, K, N = 192, 320, 512
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(K, N, device="cuda") * 0.1).to(torch.bfloat16)          # MN-major operand: out = a @ b
    src = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    groups = N // seg
    rd = torch.empty((M // seq, groups, seq) if seq else (M, groups), dtype=torch.float32, device="cuda")
    C.gemm_rowdot(a, b, True, out, src, rd, seg, seq, cuda_status)
    want = a.float() @ b.float()
    assert (out.float() - want).abs().max() < 0.02 * want.abs().max()
    dots = (out.float() * src.float()).view(M, groups, seg).sum(-1)
    if seq:
        dots = dots.view(M // seq, seq, groups).transpose(1, 2)
    assert torch.allclose(rd, dots, rtol=2e-3, atol=2e-2)


def test_batched_gemm_matches_bmm(cuda_status):
    """One launch for a stack of products, with the scaled C term used by the Newton-Schulz polynomial."""
    from forgeminds_b200 import ops
    C = ops.require()
    torch.manual_seed(3)
    G, M, N, K = 3, 256, 200, 320
    a = torch.randn(G, M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(G, N, K, device="cuda").to(torch.bfloat16)
    c = torch.randn(G, M, N, device="cuda").to(torch.bfloat16)
    tg = torch.arange(G, dtype=torch.int32, device="cuda").repeat_interleave(M // 128).contiguous()
    out = torch.empty(G, M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm_batched(a, b, out, c, False, 0.5, -2.0, tg, cuda_status)
    want = 0.5 * torch.bmm(a.float(), b.float().transpose(1, 2)) - 2.0 * c.float()
    assert (out.float() - want).norm() / want.norm() < 1e-2
    bt = b.transpose(1, 2).contiguous()                       # [G, K, N]: the MN-major form of the same operand
    C.gemm_batched(a, bt, out, None, True, 1.0, 0.0, tg, cuda_status)
    want = torch.bmm(a.float(), b.float().transpose(1, 2))
    assert (out.float() - want).norm() / want.norm() < 1e-2


@pytest.mark.parametrize("shape", [(4, 256, 384), (3, 384, 256), (1, 256, 512)])
def test_newton_schulz_stack_orthogonalises(shape, cuda_status):
    from forgeminds_b200 import kernels as K
    from forgeminds_b200.kernels import reference as _ref
    torch.manual_seed(5)
    g = torch.randn(*shape, device="cuda").to(torch.bfloat16)
    got = K.newton_schulz(g, 5)
    want = _ref.newton_schulz(g.float(), 5, torch.float32)
    assert got.shape == g.shape and got.dtype == torch.bfloat16
    assert (got.float() - want).norm() / want.norm() < 0.05
    sv = torch.linalg.svdvals(got.float())
    assert sv.min() > 0.4 and sv.max() < 1.4


@pytest.mark.parametrize("env", [{"FMB_GEMM_PAIR": "0"}, {"FMB_GEMM_DTMA": "0"}])
def test_gemm_switches_keep_the_single_cta_and_register_store_paths_correct(env):
    """The switches are read once per process, so each setting runs in a child process."""
    import os
    import subprocess
    import sys
    code = r'''
import torch
from forgeminds_b200.ops import functional as Fn
from forgeminds_b200 import ops
torch.manual_seed(0)
for (M, N, K, a_mn, b_mn, acc) in [(512, 384, 640, False, False, False), (1024, 1024, 4096, True, True, True),
                                   (304, 136, 72, True, False, False), (640, 200, 512, False, True, True)]:
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(torch.bfloat16)
    want = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    if acc:
        base = torch.randn(M, N, device="cuda")
        out = base.clone()
        Fn.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, c=out, beta=1.0, allow_split=True)
        want = want + base
    else:
        out = Fn.gemm(a, b, a_mn=a_mn, b_mn=b_mn).float()
    torch.cuda.synchronize()
    assert int(ops.status_word(torch.device("cuda")).item()) == 0
    rel = ((out - want).norm() / want.norm()).item()
    assert rel < (1e-5 if acc else 1e-2), (M, N, K, rel)
print("ok")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], env={**os.environ, **env, "PYTHONPATH": root}, capture_output=True,
                         text=True, timeout=300)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]
