"""Row kernels (norms, SwiGLU, RoPE, softmax, top-k, CE, KL, AdamW) against fp32 PyTorch."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _bf(*shape, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("d", [64, 256, 1024, 2560, 4096, 8192])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(d, wdtype):
    from forgeminds_b200.ops import functional as Fn
    x = _bf(300, d, seed=1).requires_grad_()
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(wdtype).requires_grad_()
    y = Fn.rms_norm(x, w, 1e-6)
    g = _bf(300, d, seed=2)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = F.rms_norm(xr, (d,), wr, 1e-6)
    yr.backward(g.float())
    assert (y.float() - yr).abs().max() < 0.04
    assert (x.grad.float() - xr.grad).abs().max() < 0.05
    assert (w.grad.float() - wr.grad).norm() / wr.grad.norm() < 1e-2


def test_rmsnorm_bwd_adds_the_weight_gradient_into_a_given_buffer():
    """The form the flat gradient store uses: no gradient tensor comes back, the column sum adds in place."""
    from forgeminds_b200 import ops
    C = ops.require()
    x, dy = _bf(300, 256, seed=3), _bf(300, 256, seed=4)
    w = 1 + 0.1 * torch.randn(256, device="cuda")
    _, rstd = C.rmsnorm_fwd(x, w, 1e-6)
    dx0, dw0 = C.rmsnorm_bwd(dy, x, w, rstd, None, True)
    acc = torch.full((256,), 0.5, device="cuda")
    dx1, dw1 = C.rmsnorm_bwd(dy, x, w, rstd, None, True, acc)
    assert dw1 is None and torch.equal(dx0, dx1)
    assert torch.allclose(acc, 0.5 + dw0, rtol=1e-6, atol=1e-6)


def test_rmsnorm_fp32_input():
    from forgeminds_b200.ops import functional as Fn
    x = torch.randn(77, 512, device="cuda", requires_grad=True)
    w = torch.randn(512, device="cuda", requires_grad=True)
    y = Fn.rms_norm(x, w, 1e-5)
    y.sum().backward()
    xr, wr = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    yr = F.rms_norm(xr, (512,), wr, 1e-5)
    yr.sum().backward()
    assert torch.allclose(y, yr, atol=1e-4, rtol=1e-4)
    assert torch.allclose(x.grad, xr.grad, atol=1e-4, rtol=1e-3)
    assert torch.allclose(w.grad, wr.grad, atol=1e-3, rtol=1e-3)


def test_add_rmsnorm():
    from forgeminds_b200.ops import functional as Fn
    x, dl = _bf(128, 1024, seed=3).requires_grad_(), _bf(128, 1024, seed=4).requires_grad_()
    w = torch.ones(1024, device="cuda", requires_grad=True)
    xn, y = Fn.add_rms_norm(x, dl, w, 1e-6)
    (xn.float().sum() * 0.5 + (y.float() * 0.3).sum()).backward()
    xr, dr = x.detach().float().requires_grad_(), dl.detach().float().requires_grad_()
    wr = w.detach().clone().requires_grad_()
    xnr = xr + dr
    yr = F.rms_norm(xnr, (1024,), wr, 1e-6)
    (xnr.sum() * 0.5 + (yr * 0.3).sum()).backward()
    assert (xn.float() - xnr).abs().max() < 0.03
    assert (y.float() - yr).abs().max() < 0.05
    assert (x.grad.float() - xr.grad).abs().max() < 0.02
    assert torch.equal(x.grad, dl.grad)
    assert (w.grad - wr.grad).norm() / wr.grad.norm() < 1e-2


def test_swiglu_split_and_pair():
    from forgeminds_b200.ops import functional as Fn
    gu = _bf(256, 2 * 704, seed=5).requires_grad_()
    out = Fn.swiglu_split(gu)
    g = _bf(256, 704, seed=6)
    out.backward(g)
    r = gu.detach().float().requires_grad_()
    ref = F.silu(r[:, :704]) * r[:, 704:]
    ref.backward(g.float())
    assert (out.float() - ref).abs().max() < 0.05
    assert (gu.grad.float() - r.grad).abs().max() < 0.06
    a, b = _bf(64, 128, seed=7).requires_grad_(), _bf(64, 128, seed=8).requires_grad_()
    o2 = Fn.swiglu(a, b)
    o2.sum().backward()
    assert (o2.float() - F.silu(a.detach().float()) * b.detach().float()).abs().max() < 0.05
    assert a.grad is not None and b.grad is not None


@pytest.mark.parametrize("hd", [32, 64, 80, 128])
def test_rope_qkv(hd):
    from forgeminds_b200.ops import functional as Fn
    B, T, Hq, Hkv = 2, 96, 4, 2
    qkv = _bf(B, T, (Hq + 2 * Hkv) * hd, seed=9)
    inv = 10000.0 ** (-torch.arange(0, hd, 2, device="cuda", dtype=torch.float32) / hd)
    ang = torch.outer(torch.arange(T, device="cuda", dtype=torch.float32), inv)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    ref = qkv.float().view(B, T, Hq + 2 * Hkv, hd).clone()
    rot = ref[:, :, : Hq + Hkv]
    x1, x2 = rot.chunk(2, -1)
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    ref[:, :, : Hq + Hkv] = torch.cat((x1 * c - x2 * s, x1 * s + x2 * c), -1)
    leaf = qkv.clone().requires_grad_()
    out = Fn.rope_qkv_(leaf * 1, cos, sin, Hq, Hkv, hd)
    assert (out.float().view(B, T, -1, hd) - ref).abs().max() < 0.03
    g = _bf(B, T, (Hq + 2 * Hkv) * hd, seed=10)
    out.backward(g)
    # the backward of a rotation is the inverse rotation
    gr = g.float().view(B, T, -1, hd).clone()
    g1, g2 = gr[:, :, : Hq + Hkv].chunk(2, -1)
    gr[:, :, : Hq + Hkv] = torch.cat((g1 * c + g2 * s, -g1 * s + g2 * c), -1)
    assert (leaf.grad.float().view(B, T, -1, hd) - gr).abs().max() < 0.03


def test_softmax_and_topk():
    from forgeminds_b200.ops import functional as Fn
    x = torch.randn(64, 1000, device="cuda", requires_grad=True)
    y = Fn.softmax_lastdim(x)
    (y * torch.arange(1000, device="cuda")).sum().backward()
    xr = x.detach().clone().requires_grad_()
    yr = torch.softmax(xr, -1)
    (yr * torch.arange(1000, device="cuda")).sum().backward()
    assert torch.allclose(y, yr, atol=1e-6, rtol=1e-4)
    assert torch.allclose(x.grad, xr.grad, atol=1e-4, rtol=1e-3)
    z = torch.randint(0, 50, (32, 777), device="cuda").float()      # many ties
    v, i = Fn.topk_lastdim(z, 16)
    vr, _ = torch.topk(z, 16, dim=-1)
    assert torch.equal(v, vr)
    # ties resolved towards the smaller index: indices strictly increase inside a run of equal values
    same = v[:, 1:] == v[:, :-1]
    assert bool(((i[:, 1:] > i[:, :-1]) | ~same).all())
    assert torch.equal(torch.gather(z, -1, i), v)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,k", [(32000, 64), (4096, 1), (5000, 1000), (1024, 7)])
def test_topk_radix_select(dtype, n, k):
    """The one-pass selection kernel: values as torch.topk, ties by smallest index, NaN first."""
    from forgeminds_b200.ops import functional as Fn
    g = torch.Generator(device="cuda").manual_seed(n + k)
    x = torch.randn(37, n, device="cuda", generator=g).to(dtype)
    x[1] = torch.randint(-3, 3, (n,), device="cuda", generator=g).to(dtype)      # heavy ties, negative values
    x[2] = 0                                                                       # one value only
    x[3, 17] = float("nan")
    x[4] = -x[4].abs()
    v, i = Fn.topk_lastdim(x, k)
    vr, _ = torch.topk(x.float(), k, dim=-1)
    assert torch.equal(torch.nan_to_num(v.float(), nan=1e30), torch.nan_to_num(vr, nan=1e30))
    assert torch.equal(torch.nan_to_num(torch.gather(x, -1, i).float(), nan=1e30), torch.nan_to_num(v.float(), nan=1e30))
    same = v[:, 1:] == v[:, :-1]
    assert bool(((i[:, 1:] > i[:, :-1]) | ~same).all())
    assert i[3, 0].item() == 17
    assert torch.equal(i[2], torch.arange(k, device="cuda"))


def test_cross_entropy_kernel():
    from forgeminds_b200 import ops
    C = ops.require()
    rows, V = 257, 32000
    logits = _bf(rows, V, seed=11, scale=2.0)
    labels = torch.randint(0, V, (rows,), device="cuda")
    labels[5] = -100
    ref_in = logits.float().requires_grad_()
    ref = F.cross_entropy(ref_in, labels, ignore_index=-100, reduction="sum")
    ref.backward()
    work = logits.clone()
    row_loss = C.ce_fwd_bwd(work, labels, 1.0, None, -100, True)
    assert abs(row_loss.sum().item() - ref.item()) / ref.item() < 1e-3
    assert row_loss[5] == 0
    assert (work.float() - ref_in.grad).abs().max() < 0.01
    assert work[5].abs().max() == 0


def test_linear_cross_entropy_autograd():
    from forgeminds_b200.ops import functional as Fn
    h = _bf(600, 256, seed=12).requires_grad_()
    w = (torch.randn(1024, 256, device="cuda") * 0.05).requires_grad_()
    y = torch.randint(0, 1024, (600,), device="cuda")
    y[:7] = -100
    loss = Fn.linear_cross_entropy(h, w, y, chunk=256)
    (loss * 0.5).backward()
    hr = h.detach().float().requires_grad_()
    wr = w.detach().to(torch.bfloat16).float().requires_grad_()
    lr = F.cross_entropy(hr @ wr.t(), y, ignore_index=-100)
    (lr * 0.5).backward()
    assert abs(loss.item() - lr.item()) < 2e-2
    assert (h.grad.float() - hr.grad).norm() / hr.grad.norm() < 3e-2
    assert (w.grad - wr.grad).norm() / wr.grad.norm() < 3e-2


def test_kl_kernel():
    from forgeminds_b200 import ops
    C = ops.require()
    s, t = torch.randn(33, 5000, device="cuda"), torch.randn(33, 5000, device="cuda")
    row, grad = C.kl_fwd_bwd(s, t, 1.0 / 33, True, False)
    sr = s.clone().requires_grad_()
    ref = F.kl_div(F.log_softmax(sr, -1), F.log_softmax(t, -1), reduction="batchmean", log_target=True)
    ref.backward()
    assert abs(row.sum().item() / 33 - ref.item()) < 1e-4
    assert torch.allclose(grad, sr.grad, atol=1e-6, rtol=1e-3)


def test_adamw_flat_matches_torch():
    from forgeminds_b200 import ops
    C = ops.require()
    n = 100003
    p = torch.randn(n, device="cuda")
    pr = p.clone().requires_grad_()
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    shadow = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ctl = torch.tensor([1.0, 1.0], device="cuda")
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        pr.grad = g.clone()
        opt.step()
        C.adamw_flat(p, g, m, v, shadow, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1 - 0.9 ** step, 1 - 0.95 ** step, ctl)
    assert torch.allclose(p, pr.detach(), atol=1e-5, rtol=1e-4)
    assert torch.equal(shadow, p.to(torch.bfloat16))
    before = p.clone()
    ctl[1] = 0.0                                # skip flag: nothing may change
    C.adamw_flat(p, g, m, v, shadow, 1e-2, 0.9, 0.95, 1e-8, 0.1, 0.5, 0.5, ctl)
    assert torch.equal(p, before)
    out, scratch = torch.zeros(1, device="cuda"), torch.empty(1024, device="cuda")
    C.sqnorm(g, scratch, out, False)
    assert abs(out.item() - g.double().pow(2).sum().item()) / out.item() < 1e-5


def test_router_and_moe_plan():
    from forgeminds_b200 import ops
    C = ops.require()
    rows, E, k = 1000, 8, 2
    logits = torch.randn(rows, E, device="cuda")
    probs, w, idx, lse, partial, counts = C.router_fwd(logits, k)
    pr = torch.softmax(logits, -1)
    wr, ir = pr.topk(k, -1)
    assert torch.allclose(probs, pr, atol=1e-6)
    assert torch.equal(idx.long(), ir)
    assert torch.allclose(w, wr / wr.sum(-1, keepdim=True), atol=1e-6)
    assert torch.equal(counts.long(), torch.bincount(ir.reshape(-1), minlength=E))
    assert torch.allclose(partial[:, :E].sum(0), pr.sum(0), rtol=1e-4)
    assert torch.allclose(partial[:, E].sum(), lse.pow(2).sum(), rtol=1e-4)
    slot_of, token_of, region, meta = C.moe_plan(idx, E, 128, 0, 0, rows * k + E * 128)
    flat = ir.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    start = 0
    for e in range(E):
        n_e = int((flat == e).sum())
        s0, used, padded = region[e].tolist()
        assert used == n_e and s0 == start and padded % 128 == 0
        want = order[(flat[order] == e)] // k
        assert torch.equal(token_of[s0:s0 + used].long(), want)
        start += padded
    assert int(meta) == start
    x = _bf(rows, 64, seed=13)
    xs = C.moe_gather(x, token_of)
    assert torch.equal(xs[region[0, 0]: region[0, 0] + region[0, 1]], x[token_of[: region[0, 1]].long()])
    out = C.moe_combine(xs, slot_of, w.contiguous(), rows, k)
    assert (out.float() - x.float()).abs().max() < 0.02       # weights sum to one
