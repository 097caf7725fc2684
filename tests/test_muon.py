"""Muon: param-group handling, the update rule against a hand-written statement of it, regressions."""
import pytest
import torch
import torch.nn as nn

import forgeminds_b200 as fm
from forgeminds_b200.kernels.reference import newton_schulz


def _manual_step(p, g, buf, lr, wd, mu, nesterov=True, steps=5):
    buf = buf * mu + g * (1 - mu)
    d = g * (1 - mu) + buf * mu if nesterov else buf
    o = newton_schulz(d, steps, torch.float32)
    scale = max(1.0, p.shape[0] / p.shape[1]) ** 0.5
    return p * (1 - lr * wd) - lr * scale * o, buf


def test_auto_split_and_rule():
    torch.manual_seed(0)
    lin = nn.Linear(12, 20)
    opt = fm.Muon(lin.parameters(), lr=0.05, weight_decay=0.1, ns_dtype=torch.float32)
    kinds = [g["use_muon"] for g in opt.param_groups]
    assert kinds == [True, False]
    w0 = lin.weight.detach().clone()
    lin(torch.randn(4, 12)).sum().backward()
    g = lin.weight.grad.clone()
    opt.step()
    want, _ = _manual_step(w0, g, torch.zeros_like(w0), 0.05, 0.1, 0.95)
    assert torch.allclose(lin.weight, want, atol=1e-5)
    assert torch.equal(lin.weight.grad, g)                     # the gradient itself is never modified


def test_nesterov_off_keeps_buffer_unscaled():
    w = nn.Parameter(torch.randn(30, 10))
    opt = fm.Muon([w], lr=0.01, nesterov=False, ns_dtype=torch.float32)
    for _ in range(3):
        w.grad = torch.ones_like(w)
        opt.step()
    buf = opt.state[w]["momentum_buffer"]
    assert buf.max() <= 1.0 + 1e-6                             # momentum of a constant gradient stays below it


def test_param_group_dicts_generators_and_errors():
    m = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 2))
    opt = fm.Muon((p for p in m.parameters()), lr=0.02)
    assert sum(len(g["params"]) for g in opt.param_groups) == 4
    mats = [p for p in m.parameters() if p.ndim >= 2]
    vecs = [p for p in m.parameters() if p.ndim < 2]
    opt = fm.Muon([dict(params=mats, lr=0.05, use_muon=True, extra_key=1), dict(params=vecs, use_muon=False, betas=(0.8, 0.9))])
    assert opt.param_groups[0]["extra_key"] == 1 and opt.param_groups[1]["betas"] == (0.8, 0.9)
    with pytest.raises(ValueError, match="vector"):
        fm.Muon([dict(params=vecs, use_muon=True)])
    with pytest.raises(ValueError):
        fm.Muon([])
    with pytest.raises(TypeError):
        fm.Muon([3, 4])
    with pytest.raises(ValueError):
        fm.Muon(mats, ns_steps=0)


def test_frozen_and_gradless_params():
    a, b = nn.Parameter(torch.randn(6, 6)), nn.Parameter(torch.randn(6, 6), requires_grad=False)
    c = nn.Parameter(torch.randn(6, 6))
    opt = fm.Muon([a, b, c], lr=0.02)
    a.grad = torch.randn(6, 6)
    before_b, before_c = b.clone(), c.clone()
    opt.step()
    assert torch.equal(b, before_b) and c.grad is None and b not in opt.state
    assert torch.allclose(c, before_c)                        # zero gradient: no movement (no weight decay)


def test_bucketed_equals_per_matrix_and_trains():
    torch.manual_seed(0)
    ws = [nn.Parameter(torch.randn(8, 16)) for _ in range(3)]
    ref = [w.detach().clone() for w in ws]
    opt = fm.Muon(ws, lr=0.03, ns_dtype=torch.float32)
    grads = [torch.randn(8, 16) for _ in ws]
    for w, g in zip(ws, grads):
        w.grad = g
    opt.step()
    for w, r, g in zip(ws, ref, grads):
        want, _ = _manual_step(r, g, torch.zeros_like(r), 0.03, 0.0, 0.95)
        assert torch.allclose(w, want, atol=1e-5)
    model = nn.Sequential(nn.Linear(10, 32), nn.ReLU(), nn.Linear(32, 1))
    opt = fm.Muon(model.parameters(), lr=0.02, adam_lr=1e-2)
    x, y = torch.randn(64, 10), torch.randn(64, 1)
    first = None
    for _ in range(40):
        loss = (model(x) - y).pow(2).mean()
        first = first or loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < 0.7 * first


# ------------------------------------------------------------------ the published Muon recipe as an oracle
# Keller Jordan's reference optimizer (github.com/KellerJordan/Muon, MIT licence), restated here from its
# public description: quintic Newton-Schulz with coefficients (3.4445, -4.7750, 2.0315) on the matrix scaled
# to unit Frobenius norm, iterated on the wide orientation; momentum as an exponential average; Nesterov
# blend; update scaled by sqrt(max(1, rows / cols)); decoupled weight decay.
def _kj_orthogonalize(G, steps):
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.clone()
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        A = X @ X.mT
        B = b * A + c * A @ A
        X = a * X + B @ X
    return X.mT if tall else X


def _kj_update(grad, momentum, beta=0.95, ns_steps=5, nesterov=True):
    momentum.lerp_(grad, 1 - beta)
    direction = grad.lerp(momentum, beta) if nesterov else momentum
    update = _kj_orthogonalize(direction, ns_steps)
    return update * max(1, grad.size(-2) / grad.size(-1)) ** 0.5


class _KJMuon:
    def __init__(self, params, lr, weight_decay, momentum=0.95):
        self.params, self.lr, self.wd, self.mu = list(params), lr, weight_decay, momentum
        self.bufs = [torch.zeros_like(p) for p in self.params]

    @torch.no_grad()
    def step(self):
        for p, buf in zip(self.params, self.bufs):
            update = _kj_update(p.grad, buf, beta=self.mu)
            p.mul_(1 - self.lr * self.wd)
            p.add_(update.reshape(p.shape), alpha=-self.lr)


@pytest.mark.parametrize("shape", [(24, 8), (8, 24), (16, 16)])
def test_matches_the_published_recipe_over_several_steps(shape):
    torch.manual_seed(3)
    ours = nn.Parameter(torch.randn(*shape))
    theirs = nn.Parameter(ours.detach().clone())
    a = fm.Muon([ours], lr=0.02, weight_decay=0.05, ns_dtype=torch.float32)
    b = _KJMuon([theirs], lr=0.02, weight_decay=0.05)
    for k in range(4):
        g = torch.randn(*shape, generator=torch.Generator().manual_seed(10 + k))
        ours.grad, theirs.grad = g.clone(), g.clone()
        a.step()
        b.step()
        assert torch.allclose(ours, theirs, atol=2e-5), (k, (ours - theirs).abs().max())
    assert torch.allclose(a.state[ours]["momentum_buffer"], b.bufs[0], atol=1e-6)


def test_newton_schulz_pushes_singular_values_towards_one():
    torch.manual_seed(0)
    g = torch.randn(48, 32)
    s = torch.linalg.svdvals(newton_schulz(g, 5, torch.float32))
    assert s.min() > 0.6 and s.max() < 1.25, (s.min(), s.max())          # the quintic's fixed band around 1
    assert torch.allclose(newton_schulz(g, 5, torch.float32), _kj_orthogonalize(g, 5), atol=1e-5)


def test_bf16_iteration_stays_close_to_fp32():
    torch.manual_seed(1)
    g = torch.randn(4, 32, 64)
    lo = newton_schulz(g, 5, torch.bfloat16).float()
    hi = newton_schulz(g, 5, torch.float32)
    assert (lo - hi).norm() / hi.norm() < 0.05


def test_device_side_skip_and_clip(monkeypatch):
    """``step(ctl=...)``: gradients are scaled by ctl[0]; with ctl[1] = 0 nothing moves, even when the
    gradient is not finite."""
    torch.manual_seed(0)
    w, v = nn.Parameter(torch.randn(8, 16)), nn.Parameter(torch.randn(16))
    opt = fm.Muon([w, v], lr=0.05, ns_dtype=torch.float32)
    w.grad, v.grad = torch.randn(8, 16), torch.randn(16)
    opt.step(ctl=torch.tensor([1.0, 1.0]))
    snap = [t.clone() for t in (w, v, opt.state[w]["momentum_buffer"], opt.state[v]["exp_avg"])]
    w.grad, v.grad = torch.full((8, 16), float("nan")), torch.full((16,), float("inf"))
    opt.step(ctl=torch.tensor([1.0, 0.0]))
    now = (w, v, opt.state[w]["momentum_buffer"], opt.state[v]["exp_avg"])
    assert all(torch.equal(a, b.detach()) for a, b in zip(snap, now))
    # a clip coefficient scales what the AdamW group sees exactly like scaling its gradient would
    a, b = nn.Parameter(torch.ones(16)), nn.Parameter(torch.ones(16))
    oa, ob = fm.Muon([a], lr=0.05), fm.Muon([b], lr=0.05)
    g = torch.randn(16)
    a.grad, b.grad = g.clone(), g * 0.25
    oa.step(ctl=torch.tensor([0.25, 1.0]))
    ob.step()
    assert torch.allclose(a, b, atol=1e-7) and torch.allclose(oa.state[a]["exp_avg"], ob.state[b]["exp_avg"])


def test_two_ranks_share_the_newton_schulz_work():
    """2 Gloo ranks under torchrun: see tests/muon_mp_check.py."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29644", os.path.join(here, "muon_mp_check.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0 and "MUON_MP_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-4000:]
