"""The reference package as a black-box oracle on CPU: same names, same numbers.

Runs when the unmodified reference is installed under ``baseline/_ref`` (the benchmark's reference
arm uses the same copy); skipped otherwise.
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "forgemind")),
                                reason="reference package not installed under baseline/_ref")


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, REF)
    try:
        import forgemind
        yield forgemind
    finally:
        sys.path.remove(REF)


def _cfg(mod, **over):
    base = dict(vocab_size=256, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=32)
    base.update(over)
    return mod.GPTConfig(**base)


def test_public_names_match(ref):
    import forgeminds_b200 as fm
    missing = [n for n in ref.__all__ if not hasattr(fm, n)]
    assert not missing, missing
    assert not hasattr(fm, "Fabric")


def test_config_fields_are_a_superset(ref):
    import dataclasses
    import forgeminds_b200 as fm
    for name in ("ParallelConfig", "QuantConfig", "OffloadConfig", "TrainConfig", "GPTConfig"):
        theirs = {f.name: f.default for f in dataclasses.fields(getattr(ref, name))}
        ours = {f.name: f.default for f in dataclasses.fields(getattr(fm, name))}
        assert set(theirs) <= set(ours), (name, sorted(set(theirs) - set(ours)))
        for key, default in theirs.items():
            if default is dataclasses.MISSING or isinstance(default, (list, tuple, dict)):
                continue
            assert ours[key] == default, (name, key, ours[key], default)


@pytest.mark.parametrize("over", [dict(), dict(tie_embeddings=True), dict(n_experts=4, top_k=2, moe_every=1)])
def test_gpt_state_dict_and_outputs_match(ref, over):
    import forgeminds_b200 as fm
    torch.manual_seed(0)
    theirs = ref.GPT(_cfg(ref, **over)).eval()
    ours = fm.GPT(_cfg(fm, **over)).eval()
    assert list(theirs.state_dict().keys()) == list(ours.state_dict().keys())
    assert [tuple(v.shape) for v in theirs.state_dict().values()] == [tuple(v.shape) for v in ours.state_dict().values()]
    ours.load_state_dict(theirs.state_dict())
    tok = torch.randint(0, 256, (3, 32))
    lab = torch.randint(0, 256, (3, 32))
    with torch.no_grad():
        assert torch.allclose(ours(tok), theirs(tok), atol=1e-5, rtol=1e-5)
    lo, ao = ours(tok, labels=lab)
    lt, at = theirs(tok, labels=lab)
    assert torch.allclose(lo, lt, atol=1e-5)
    if at is not None:
        assert torch.allclose(ao, at, atol=1e-5)
    (lo + (ao if ao is not None else 0)).backward()
    (lt + (at if at is not None else 0)).backward()
    for (n1, p1), (n2, p2) in zip(ours.named_parameters(), theirs.named_parameters()):
        assert n1 == n2
        assert torch.allclose(p1.grad, p2.grad, atol=2e-5, rtol=1e-4), n1
    assert ours.num_params() == theirs.num_params()
    assert ours.flops_per_token(32) == theirs.flops_per_token(32)


def test_kernel_functions_match_the_reference_fallback(ref):
    import forgeminds_b200 as fm
    rk, ok = ref.kernels, fm.kernels
    torch.manual_seed(1)
    x, w, d = torch.randn(7, 48), torch.rand(48) + 0.5, torch.randn(7, 48)
    assert torch.allclose(ok.rms_norm(x, w, 1e-6), rk.rms_norm(x, w, 1e-6), atol=1e-6)
    a, b = ok.add_rms_norm(x, d, w, 1e-6), rk.add_rms_norm(x, d, w, 1e-6)
    assert torch.allclose(a[0], b[0]) and torch.allclose(a[1], b[1], atol=1e-6)
    g, u = torch.randn(5, 24), torch.randn(5, 24)
    assert torch.allclose(ok.swiglu(g, u), rk.swiglu(g, u), atol=1e-6)
    z = torch.randint(0, 5, (4, 40)).float()
    vo, io = ok.topk(z, 6)
    vt, it = rk.topk(z, 6)
    assert torch.equal(vo, vt) and torch.equal(torch.gather(z, -1, io), vt)     # their CPU path leaves tie order to torch.topk
    s = torch.randn(6, 33)
    assert torch.allclose(ok.softmax(s), rk.softmax(s), atol=1e-6)


def test_chunked_cross_entropy_matches(ref):
    from forgeminds_b200.loss import chunked_cross_entropy as ours
    theirs = ref.loss.chunked_cross_entropy
    torch.manual_seed(2)
    h, w = torch.randn(2, 9, 16, requires_grad=True), torch.randn(50, 16, requires_grad=True)
    y = torch.randint(0, 50, (2, 9))
    y[0, 3] = -100
    h2, w2 = h.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    a, b = ours(h, w, y, 4), theirs(h2, w2, y, 4)
    assert torch.allclose(a, b, atol=1e-6)
    a.backward()
    b.backward()
    assert torch.allclose(h.grad, h2.grad, atol=1e-6) and torch.allclose(w.grad, w2.grad, atol=1e-6)


def test_lr_schedule_and_step_metrics_match(ref, tmp_path):
    import forgeminds_b200 as fm
    outs = {}
    for name, mod in (("ours", fm), ("theirs", ref)):
        torch.manual_seed(0)
        cfg = mod.ForgeConfig()
        cfg.train.max_steps, cfg.train.warmup_steps, cfg.train.lr = 6, 2, 1e-2
        cfg.train.bf16, cfg.train.resume, cfg.train.log_every = False, False, 1000
        cfg.train.ckpt_dir = str(tmp_path / name)
        tr = mod.Trainer(lambda ctx: mod.GPT(_cfg(mod)), cfg, mod.SyntheticLM(256, 32, n=64), micro_batch=4)
        hist = tr.fit()
        if hasattr(tr, "close"):
            tr.close()
        outs[name] = hist
    for a, b in zip(outs["ours"], outs["theirs"]):
        assert set(b) <= set(a)
        assert a["lr"] == pytest.approx(b["lr"], rel=1e-9)
        assert a["loss"] == pytest.approx(b["loss"], abs=2e-4)
        assert a["grad_norm"] == pytest.approx(b["grad_norm"], rel=2e-3)
