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
