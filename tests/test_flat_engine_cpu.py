"""The flat-store engine's bookkeeping on CPU (PyTorch operators stand in for the sm_100a kernels).

``FORGEMINDS_FLAT_ENGINE=1`` selects the engine without a GPU. Checked here: it follows the library
engine step for step (AdamW and Muon, with clipping active), a non-finite step leaves weights and
optimizer state untouched although the update is enqueued before the host reads the flag, and a Muon
run resumes exactly from a checkpoint.
"""
import os

import pytest
import torch

import forgeminds_b200 as fm


@pytest.fixture
def flat_env(monkeypatch):
    def use(flat: bool):
        monkeypatch.setenv("FORGEMINDS_FLAT_ENGINE", "1" if flat else "0")
    return use


def _trainer(optimizer, steps, ckpt_dir="unused", resume=False, clip=0.5):
    cfg = fm.ForgeConfig()
    cfg.train.__dict__.update(max_steps=steps, bf16=False, log_every=1000, warmup_steps=2, lr=3e-3, resume=resume,
                              prefetch=False, optimizer=optimizer, grad_clip=clip, ckpt_dir=ckpt_dir, ckpt_every=0)
    mc = fm.GPTConfig(vocab_size=256, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=32, native=False)
    return fm.Trainer(lambda c: fm.GPT(mc), cfg, fm.SyntheticLM(256, 32, n=512), micro_batch=8)


def _losses(tr, n):
    out = [tr.train_step()["loss"] for _ in range(n)]
    return out


@pytest.mark.parametrize("optimizer", ["adamw", "muon"])
def test_flat_engine_follows_the_library_engine(flat_env, optimizer):
    flat_env(True)
    a = _trainer(optimizer, 6)
    assert a.eng.name == "native" and a.store is not None
    la = _losses(a, 6)
    a.close()
    flat_env(False)
    b = _trainer(optimizer, 6)
    assert b.eng.name == "library"
    lb = _losses(b, 6)
    b.close()
    assert max(abs(x - y) for x, y in zip(la, lb)) < 2e-4, (la, lb)
    assert la[-1] < la[0]


@pytest.mark.parametrize("optimizer", ["adamw", "muon"])
def test_nonfinite_step_is_not_applied(flat_env, optimizer):
    flat_env(True)
    tr = _trainer(optimizer, 5)
    _losses(tr, 2)
    honest = tr._clip

    def poisoned():
        honest()
        tr.store.grad.fill_(float("nan"))          # what a real overflow leaves behind
        return torch.tensor(float("nan"))
    tr._clip = poisoned
    before = tr.store.master.clone()
    state_before = None
    if tr.eng.muon is not None:
        state_before = [v.clone() for st in tr.eng.muon.state.values() for v in st.values() if torch.is_tensor(v)]
    m = tr.train_step()
    tr._clip = honest
    assert m["skipped"] == 1
    assert torch.equal(before, tr.store.master), "a skipped step moved the weights"
    if state_before is not None:
        after = [v for st in tr.eng.muon.state.values() for v in st.values() if torch.is_tensor(v)]
        assert all(torch.equal(x, y) for x, y in zip(state_before, after)), "a skipped step moved the Muon state"
    more = tr.train_step()
    assert more["loss"] == more["loss"] and more["skipped"] == 1
    tr.close()


def test_muon_clip_coefficient_reaches_the_update(flat_env):
    """With a tiny clip threshold the update shrinks for the AdamW group (Muon's orthogonalised update is
    scale-free, its momentum is not): the two engines still agree, which they only do when the flat
    engine hands ``ctl[0]`` to Muon."""
    flat_env(True)
    a = _trainer("muon", 4, clip=0.01)
    la = _losses(a, 4)
    a.close()
    flat_env(False)
    b = _trainer("muon", 4, clip=0.01)
    lb = _losses(b, 4)
    b.close()
    assert max(abs(x - y) for x, y in zip(la, lb)) < 2e-4, (la, lb)


def test_muon_run_resumes_exactly(flat_env, tmp_path):
    flat_env(True)
    whole = _trainer("muon", 6)
    want = _losses(whole, 6)
    whole.close()
    first = _trainer("muon", 6, ckpt_dir=str(tmp_path))
    got = _losses(first, 3)
    first.save()
    first.close()
    second = _trainer("muon", 6, ckpt_dir=str(tmp_path), resume=True)
    assert second.step == 3
    got += _losses(second, 3)
    second.close()
    assert got == want, (got, want)
