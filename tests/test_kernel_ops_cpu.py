"""The `torch.library` forms of the kernels: equal to the eager path, traceable, visible in an export.

Counterpart of the reference's `tests/test_kernel_ops.py`.
"""
import pytest
import torch

import forgeminds_b200 as fm

K = fm.kernels


@pytest.fixture
def ops_on():
    K.use_custom_ops(True)
    yield
    K.use_custom_ops(False)


def _inputs():
    torch.manual_seed(0)
    x = torch.randn(4, 6, 32, requires_grad=True)
    d = torch.randn(4, 6, 32, requires_grad=True)
    w = torch.randn(32, requires_grad=True)
    return x, d, w


def _grads(fn, leaves):
    out = fn()
    out = out if isinstance(out, tuple) else (out,)
    loss = sum((o * torch.arange(o.numel(), dtype=o.dtype).view_as(o)).sum() for o in out)
    return [o.detach() for o in out], torch.autograd.grad(loss, leaves)


def test_custom_ops_equal_the_eager_functions(ops_on):
    x, d, w = _inputs()
    cases = [(lambda: K.rms_norm(x, w, 1e-5), (x, w)), (lambda: K.add_rms_norm(x, d, w, 1e-5), (x, d, w)),
             (lambda: K.swiglu(x, d), (x, d))]
    for make, leaves in cases:
        K.use_custom_ops(False)
        eo, eg = _grads(make, leaves)
        K.use_custom_ops(True)
        co, cg = _grads(make, leaves)
        for a, b in zip(eo + list(eg), co + list(cg)):
            assert torch.allclose(a, b, rtol=1e-4, atol=1e-3 * float(a.abs().max()))


def test_fake_implementations_agree_on_shape_and_dtype(ops_on):
    from torch._subclasses.fake_tensor import FakeTensorMode
    x, d, w = (t.detach() for t in _inputs())
    real = (K.rms_norm(x, w), *K.add_rms_norm(x, d, w), K.swiglu(x, d))
    with FakeTensorMode() as mode:
        fx, fd, fw = (mode.from_tensor(t) for t in (x, d, w))
        fake = (K.rms_norm(fx, fw), *K.add_rms_norm(fx, fd, fw), K.swiglu(fx, fd))
    for r, f in zip(real, fake):
        assert r.shape == f.shape and r.dtype == f.dtype


def test_fullgraph_compile_forward_and_backward(ops_on):
    x, d, w = _inputs()

    def f(x, d, w):
        s, y = K.add_rms_norm(x, d, w, 1e-5)
        return (K.swiglu(y, s) + K.rms_norm(s, w, 1e-5)).sum()

    want = torch.autograd.grad(f(x, d, w), (x, d, w))
    got = torch.autograd.grad(torch.compile(f, fullgraph=True, backend="aot_eager")(x, d, w), (x, d, w))
    for a, b in zip(want, got):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-5)


def test_export_shows_the_ops(ops_on):
    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.ones(32))

        def forward(self, x):
            return K.swiglu(K.rms_norm(x, self.w, 1e-5), x)

    text = str(torch.export.export(M(), (torch.randn(2, 32),)).graph)
    assert "forgeminds_b200.rms_norm.default" in text and "forgeminds_b200.swiglu.default" in text


def test_environment_switch(monkeypatch):
    from forgeminds_b200.kernels import _ops
    monkeypatch.setenv("FORGEMINDS_KERNEL_OPS", "1")
    assert _ops.env_default()
    monkeypatch.delenv("FORGEMINDS_KERNEL_OPS")
    assert not _ops.env_default()
