"""Forge facade: accumulation, host-read budget, clipping, checkpoints, callbacks, skip paths."""
import math

import pytest
import torch
import torch.nn as nn

import forgeminds_b200 as fm


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 1))


def _batches(n, bs=4):
    g = torch.Generator().manual_seed(1)
    return [(torch.randn(bs, 8, generator=g), torch.randn(bs, 1, generator=g)) for _ in range(n)]


def _loss(out, batch):
    return nn.functional.mse_loss(out, batch[1])


def _forge(model, **kw):
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    kw.setdefault("precision", "fp32")
    kw.setdefault("quiet", True)
    kw.setdefault("async_batches", False)
    return fm.Forge(model, opt, loss_fn=_loss, forward_fn=lambda m, b: m(b[0]), **kw)


def test_accumulation_equals_big_batch():
    data = _batches(2)
    a, b = _model(), _model()
    fa = _forge(a, accum=2, clip=0)
    assert fa.step(data[0]) is None
    st = fa.step(data[1])
    assert isinstance(st, fm.forge.ForgeState) and st.step == 1 and math.isnan(st.grad_norm)
    big = (torch.cat([data[0][0], data[1][0]]), torch.cat([data[0][1], data[1][1]]))
    _forge(b, accum=1, clip=0).step(big)
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert torch.allclose(pa, pb, atol=1e-6)


def test_one_host_read_per_update():
    f = _forge(_model(), accum=2)
    data = _batches(4)
    with fm.count_host_syncs(count_cpu=True) as c:
        for b in data:
            f.step(b)
    assert c.own == 2, c.report()


def test_clip_bounds_the_update():
    m = _model()
    f = _forge(m, clip=1e-3)
    st = f.step(_batches(1)[0])
    assert st.grad_norm > 1e-3


def test_save_load_roundtrip(tmp_path):
    f = _forge(_model(), schedule="cosine", max_steps=10)
    for b in _batches(3):
        f.step(b)
    path = str(tmp_path / "ck" / "forge.pt")
    f.save(path)
    blob = torch.load(path, weights_only=False)
    assert set(blob) == {"model", "optimizer", "scheduler", "step", "ema_loss", "rng"}
    assert all(not k.startswith("module.") for k in blob["model"])
    g = _forge(_model(), schedule="cosine", max_steps=10).load(path)
    assert g.step_count == 3
    for pa, pb in zip(f.raw_model.parameters(), g.raw_model.parameters()):
        assert torch.equal(pa, pb)


def test_fit_epochs_callbacks_and_history():
    seen = []

    class CB:
        def on_step(self, forge, state):
            seen.append(state.step)

        def on_epoch(self, forge, epoch):
            seen.append(("epoch", epoch))
    f = _forge(_model(), callbacks=[CB()], async_batches=True)
    hist = f.fit(_batches(3), max_steps=100, epochs=2)
    assert len(hist) == 6 and seen.count(("epoch", 0)) == 1 and seen.count(("epoch", 1)) == 1
    assert f.evaluate(_batches(2)) > 0


def test_nonfinite_and_spike_skips():
    f = _forge(_model(), skip_spike_factor=2.0)
    data = _batches(3)
    assert f.step(data[0]).skipped is False
    bad = (data[1][0], data[1][1] * float("nan"))
    st = f.step(bad)
    assert st.skipped and f.step_count == 1
    spike = (data[2][0], data[2][1] * 1e6)
    assert f.step(spike).skipped


def test_loss_extraction_rules():
    class Dicty(nn.Module):
        def __init__(self):
            super().__init__()
            self.l = nn.Linear(8, 1)

        def forward(self, x, y):
            return {"loss": (self.l(x) - y).pow(2).mean()}
    f = fm.Forge(Dicty(), None, precision="fp32", quiet=True, async_batches=False)
    assert f.step({"x": torch.randn(2, 8), "y": torch.randn(2, 1)}).step == 1
    with pytest.raises(ValueError):
        fm.Forge(_model(), None, precision="fp8")
    with pytest.raises(ValueError):
        fm.Forge(_model(), None, accum=0)
    with pytest.raises(ValueError):
        fm.Forge(_model(), None, offload="everything")
    assert "Forge(" in repr(f)


def test_launch_spawns_ranks_that_train_identical_replicas():
    """``fm.launch(nproc=2)`` on CPU: see tests/forge_mp_check.py."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK", "MASTER_PORT"):
        env.pop(k, None)
    out = subprocess.run([sys.executable, os.path.join(here, "forge_mp_check.py"), "29643"], capture_output=True,
                         text=True, timeout=300, env=env)
    assert out.returncode == 0 and "FORGE_MP_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-4000:]
