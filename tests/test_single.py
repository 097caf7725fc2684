"""End-to-end single-process training on CPU (the library engine)."""
import copy
import os

import pytest
import torch

import forgeminds_b200 as fm


def _cfg(tmp_path=None, **over):
    cfg = fm.ForgeConfig()
    cfg.train.__dict__.update(max_steps=40, bf16=False, log_every=1000, warmup_steps=5, lr=3e-3, resume=False,
                              prefetch=False)
    if tmp_path is not None:
        cfg.train.ckpt_dir = str(tmp_path / "ckpt")
    cfg.train.__dict__.update(over)
    return cfg


def _mc(**over):
    base = dict(vocab_size=256, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=32)
    base.update(over)
    return fm.GPTConfig(**base)


def _train(cfg, mc, moe=False, micro_batch=8):
    ds = fm.SyntheticLM(mc.vocab_size, mc.max_seq, n=512)
    tr = fm.Trainer(lambda ctx: fm.GPT(mc, fm.moe_kwargs(ctx, cfg) if moe else None), cfg, ds, micro_batch=micro_batch)
    hist = tr.fit()
    tr.close()
    return tr, hist


def test_dense_loss_drops():
    _, h = _train(_cfg(), _mc())
    assert h[-1]["loss"] < 0.6 * h[0]["loss"]
    assert set(h[0]) >= {"step", "loss", "lr", "grad_norm", "dt", "skipped", "tok_s"}


def test_moe_and_accumulation():
    _, h = _train(_cfg(grad_accum=2), _mc(n_experts=4, top_k=2), moe=True)
    assert h[-1]["loss"] < 0.6 * h[0]["loss"]


def test_moe_capacity_factor_trains():
    _, h = _train(_cfg(), _mc(n_experts=4, top_k=2, capacity_factor=1.25), moe=True)
    assert h[-1]["loss"] < 0.7 * h[0]["loss"]


@pytest.mark.parametrize("ac", ["full", "selective"])
def test_activation_checkpointing_matches_plain(ac):
    _, a = _train(_cfg(max_steps=5), _mc())
    _, b = _train(_cfg(max_steps=5, ac=ac), _mc())
    assert abs(a[-1]["loss"] - b[-1]["loss"]) < 1e-4


def test_offloaded_adamw_matches_adamw():
    _, a = _train(_cfg(max_steps=8), _mc())
    cfg = _cfg(max_steps=8)
    cfg.offload.optimizer, cfg.offload.smart = True, False
    _, b = _train(cfg, _mc())
    assert abs(a[-1]["loss"] - b[-1]["loss"]) < 1e-4


def test_expert_offload_uses_parameter_lists():
    cfg = _cfg(max_steps=3)
    cfg.offload.experts = True
    tr, _ = _train(cfg, _mc(n_experts=4), moe=True)
    keys = list(tr.raw.state_dict())
    assert any(k.endswith("experts.w1.0") for k in keys)


def test_checkpoint_resume_is_exact(tmp_path):
    cfg = _cfg(tmp_path, max_steps=6, ckpt_every=3, resume=True)
    tr, _ = _train(cfg, _mc())
    final = {k: v.clone() for k, v in tr.raw.state_dict().items()}
    # start again from the step-3 checkpoint and run to step 6
    root = cfg.train.ckpt_dir
    with open(os.path.join(root, "latest"), "w") as f:
        f.write("step_0000003")
    tr2, _ = _train(_cfg(tmp_path, max_steps=6, ckpt_every=0, resume=True), _mc())
    assert tr2.step == 6
    for k, v in tr2.raw.state_dict().items():
        assert torch.equal(v, final[k]), k
    assert os.path.exists(os.path.join(root, "step_0000006", "meta_rank0.json"))


def test_nonfinite_step_is_skipped():
    cfg = _cfg(max_steps=4)
    mc = _mc()
    ds = fm.SyntheticLM(mc.vocab_size, mc.max_seq, n=256)
    tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, ds, micro_batch=8)
    before = copy.deepcopy(tr.raw.state_dict())
    real = tr._clip
    tr._clip = lambda: torch.tensor(float("nan"))
    m = tr.train_step()
    assert m["skipped"] == 1
    for k, v in tr.raw.state_dict().items():
        assert torch.equal(v, before[k])
    tr._clip = real
    assert tr.train_step()["skipped"] == 1
    tr.close()


def test_muon_inside_trainer():
    _, h = _train(_cfg(optimizer="muon", max_steps=30, muon_lr=0.02), _mc())
    assert h[-1]["loss"] < 0.8 * h[0]["loss"]


def test_explicit_ffn_hidden():
    m = fm.GPT(_mc(dim=256, ffn_hidden=688, n_heads=8, n_kv_heads=2))
    assert m.layers["0"].ffn.w1.weight.shape == (688, 256)
    assert fm.GPT(_mc(dim=256, n_heads=8)).layers["0"].ffn.w1.weight.shape[0] == 704


def test_flops_and_params_follow_reference_formula():
    # flagship config: 336 118 784 parameters, 2 620 692 480 FLOPs per token at seq 2048
    mc = fm.GPTConfig(vocab_size=32000, dim=1024, n_layers=24, n_heads=16, n_kv_heads=4, ffn_hidden=2816, max_seq=2048)
    with torch.device("meta"):
        m = fm.GPT(mc)
    assert m.num_params() == 336118784
    assert m.flops_per_token(2048) == 2620692480


def test_config_check_names_the_offending_field():
    """A misspelt mode or an impossible mesh is reported by field name before anything is built."""
    import pytest
    good = fm.ForgeConfig()
    good.parallel.dp_shard = -1
    assert good.check(8) is good
    for change, world, needle in (
            (lambda c: setattr(c.train, "ac", "selectiv"), None, "train.ac"),
            (lambda c: setattr(c.train, "optimizer", "lion"), None, "train.optimizer"),
            (lambda c: setattr(c.train, "grad_accum", 0), None, "train.grad_accum"),
            (lambda c: setattr(c.quant, "mode", "fp4"), None, "quant.mode"),
            (lambda c: setattr(c.offload, "act_layers", 1.5), None, "offload.act_layers"),
            (lambda c: setattr(c.parallel, "pp_schedule", "zero-bubble"), None, "parallel.pp_schedule"),
            (lambda c: setattr(c.parallel, "tp", 3), 8, "does not divide"),
            (lambda c: (setattr(c.parallel, "dp_shard", 8), setattr(c.parallel, "ep", 3)), 8, "parallel.ep")):
        cfg = fm.ForgeConfig()
        change(cfg)
        with pytest.raises(ValueError, match=needle):
            cfg.check(world)
    bad = fm.ForgeConfig()
    bad.train.ac = "sometimes"
    with pytest.raises(ValueError, match="train.ac"):
        fm.Trainer(lambda ctx: None, bad, fm.SyntheticLM(64, 8, n=8))
