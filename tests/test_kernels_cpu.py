"""The PyTorch statements of the kernels (CPU path of fm.kernels) against plain torch, with gradients."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import forgeminds_b200 as fm

K = fm.kernels


def test_rms_norm_matches_torch_and_gradcheck():
    x, w = torch.randn(5, 48), torch.randn(48)
    assert torch.allclose(K.rms_norm(x, w, 1e-6), F.rms_norm(x, (48,), w, 1e-6), atol=1e-6)
    xd = torch.randn(3, 8, dtype=torch.float64, requires_grad=True)
    wd = torch.randn(8, dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(lambda a, b: K.rms_norm(a, b, 1e-6), (xd, wd))
    half = K.rms_norm(x.bfloat16(), w.bfloat16())
    assert half.dtype == torch.bfloat16


def test_add_rms_norm_returns_sum_and_norm():
    x, d, w = torch.randn(4, 32), torch.randn(4, 32), torch.randn(32)
    xn, y = K.add_rms_norm(x, d, w)
    assert torch.allclose(xn, x + d) and torch.allclose(y, F.rms_norm(x + d, (32,), w, 1e-6), atol=1e-6)


def test_swiglu_variants():
    g, u = torch.randn(6, 40), torch.randn(6, 40)
    assert torch.allclose(K.swiglu(g, u), F.silu(g) * u, atol=1e-6)
    assert torch.allclose(K.swiglu_split(torch.cat([g, u], -1)), F.silu(g) * u, atol=1e-6)
    gd = torch.randn(2, 6, dtype=torch.float64, requires_grad=True)
    ud = torch.randn(2, 6, dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(K.swiglu, (gd, ud))


def test_qk_norm_rope_odd_head_dim_and_noncontiguous():
    B, T, H, D = 2, 5, 3, 6
    x = torch.randn(B, H, T, D).transpose(1, 2)
    w = torch.randn(D)
    ang = torch.outer(torch.arange(T).float(), 10000.0 ** (-torch.arange(0, D, 2).float() / D))
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    y = K.qk_norm_rope(x, w, cos, sin)
    n = F.rms_norm(x, (D,), w, 1e-6)
    a, b = n.chunk(2, -1)
    assert torch.allclose(y, torch.cat((a * cos - b * sin, a * sin + b * cos), -1), atol=1e-5)


def test_kl_div_and_distill():
    s, t = torch.randn(7, 50, requires_grad=True), torch.randn(7, 50)
    loss = K.kl_div_logits(s, t)
    ref = F.kl_div(F.log_softmax(s, -1), F.log_softmax(t, -1), reduction="batchmean", log_target=True)
    assert torch.allclose(loss, ref, atol=1e-6)
    assert K.kl_div is K.kl_div_logits and K.distill_kl is K.kl_distill_loss
    with pytest.raises(ValueError):
        K.kl_div_logits(s, t, reduction="median")
    hs, ht = torch.randn(9, 16, requires_grad=True), torch.randn(9, 16)
    w, head = torch.randn(50, 16, requires_grad=True), nn.Linear(16, 50)
    out = K.kl_distill_loss(hs, ht, w, head, chunk=4)
    want = F.kl_div(F.log_softmax(hs @ w.t(), -1), F.log_softmax(head(ht), -1), reduction="batchmean", log_target=True)
    assert torch.allclose(out, want, atol=1e-5)
    out.backward()
    assert hs.grad is not None and head.weight.grad is None


def test_newton_schulz_orthogonalises():
    g = torch.randn(2, 24, 40)
    o = K.newton_schulz(g, steps=5, dtype=torch.float32)
    sv = torch.linalg.svdvals(o)
    assert sv.min() > 0.5 and sv.max() < 1.3
    tall = K.newton_schulz(torch.randn(40, 24), 5, dtype=torch.float32)
    assert tall.shape == (40, 24)
    with pytest.raises(ValueError):
        K.newton_schulz(torch.randn(5))
    with pytest.raises(ValueError):
        K.newton_schulz(g, steps=0)


def test_topk_ties_nan_and_errors():
    x = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0], [float("nan"), 0.0, 5.0, 5.0, -1.0]])
    v, i = K.topk(x, 3)
    assert i[0].tolist() == [1, 2, 4]
    assert i[1].tolist() == [0, 2, 3] and torch.isnan(v[1, 0])
    with pytest.raises(RuntimeError):
        K.topk(x, 9)
    vals, idx = K.topk(torch.randn(4, 6, 9), 2, dim=1)
    assert vals.shape == (4, 2, 9)
    y = torch.randn(3, 10, requires_grad=True)
    K.topk(y, 2)[0].sum().backward()
    assert y.grad.abs().sum() == 2 * 3


def test_softmax_matches_torch():
    x = torch.randn(4, 33, requires_grad=True)
    assert torch.allclose(K.softmax(x), torch.softmax(x, -1))
    assert torch.allclose(K.softmax(x, dim=0), torch.softmax(x, 0))
    assert K.softmax(x.detach().half(), dtype=torch.float32).dtype == torch.float32


def test_backend_switch_and_stats():
    K.reset_stats()
    K.set_backend("fallback")
    K.rms_norm(torch.randn(2, 8), torch.ones(8))
    st = K.stats()
    assert st["fallback"] >= 1 and "backend=fallback" in st["reasons"]
    K.set_backend("auto")
    assert K.get_backend() == "auto"
    K.set_backend("triton")
    assert K.get_backend() == "native"
    K.set_backend("auto")
    with pytest.raises(ValueError):
        K.set_backend("fast")
    assert K.HAS_TRITON is False and K.available() in (True, False)


class _Norm(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(d)), 1e-6

    def forward(self, x):
        return x * 2


class _MLP(nn.Module):
    def __init__(self, d, h):
        super().__init__()
        self.w1, self.w3, self.w2 = nn.Linear(d, h, bias=False), nn.Linear(d, h, bias=False), nn.Linear(h, d, bias=False)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


def test_patch_enable_revert():
    model = nn.Sequential(fm.models.gpt.RMSNorm(16), _MLP(16, 32), nn.RMSNorm(16))
    x = torch.randn(3, 16)
    before = model(x)
    K.enable(model)
    assert model._fm_fused == {"norm": 2, "mlp": 1}
    assert torch.allclose(model(x), before, atol=1e-6)
    assert K.patch(model[0]) is True                     # idempotent
    K.revert(model)
    assert model._fm_fused_reverted["restored"] == 3 and "forward" not in model[1].__dict__
    assert K.patch(nn.Linear(4, 4)) is False
    odd = _Norm(16)
    assert K.patch(odd) is False and K.patch(odd, kind="norm") is True
    assert torch.allclose(odd(x), F.rms_norm(x, (16,), odd.weight, 1e-6), atol=1e-6)
    with pytest.raises(TypeError):
        K.patch(nn.Linear(4, 4), kind="mlp")
    with pytest.raises(ValueError):
        K.patch(_Norm(16), kind="attention")
    mlp = _MLP(16, 32)
    want = mlp(x)
    assert K.patch(mlp, split=True) and hasattr(mlp, "gate_up") and not hasattr(mlp, "w1")
    assert torch.allclose(mlp(x), want, atol=1e-6)
    K.revert(mlp)
    assert mlp._fm_fused_reverted == {"restored": 0, "structural": 1}


def test_nn_blocks():
    norm = fm.nn.RMSNorm(24)
    x = torch.randn(2, 5, 24)
    assert torch.allclose(norm(x), nn.RMSNorm(24, eps=1e-6)(x), atol=1e-6)
    normed, res = norm.forward_with_residual(x, x)
    assert torch.allclose(res, 2 * x)
    with pytest.raises(ValueError):
        norm(torch.randn(2, 7))
    with pytest.raises(ValueError):
        norm.forward_with_residual(x, torch.randn(1, 24))
    nn.RMSNorm(24).load_state_dict(norm.state_dict())
    mlp = fm.nn.SwiGLU(24, 40)
    want = mlp(x)
    assert torch.allclose(mlp.to_split(inplace=False)(x), want, atol=1e-6)
    assert torch.allclose(mlp.to_split()(x), want, atol=1e-6) and "gate_up.weight" in mlp.state_dict()
    with pytest.raises(ValueError):
        fm.nn.RMSNorm(0)
