"""Public surface, world-1 collectives, seeding, lazy imports."""
import subprocess
import sys

import pytest
import torch

import forgeminds_b200 as fm


def test_public_names_resolve():
    for name in fm.__all__:
        assert getattr(fm, name) is not None, name
    assert not hasattr(fm, "Fabric")
    for sub in ("kernels", "autotune", "nn", "muon"):
        assert getattr(fm, sub).__name__.endswith(sub)


def test_world_one_collectives_are_identity():
    t = torch.arange(4.0)
    assert fm.all_reduce(t) is t
    assert fm.all_reduce(t, "sum") is t
    assert fm.broadcast(t) is t
    assert fm.all_gather(t) is t
    fm.barrier()
    with pytest.raises(KeyError):
        fm.all_reduce(t, "median")


def test_seed_everything_is_reproducible():
    assert fm.seed_everything(7) == 7
    a = torch.rand(3)
    fm.seed_everything(7)
    assert torch.equal(a, torch.rand(3))


def test_import_is_light():
    code = ("import sys, forgeminds_b200 as fm\n"
            "bad = [m for m in ('forgeminds_b200.kernels', 'forgeminds_b200._C', 'triton', 'torch._dynamo') if m in sys.modules]\n"
            "assert not bad, bad\n"
            "fm.kernels; assert 'forgeminds_b200.kernels' in sys.modules\n")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=".")
    assert out.returncode == 0, out.stderr


def test_config_defaults_match_reference_values():
    c = fm.ForgeConfig()
    assert (c.train.lr, c.train.betas, c.train.eps, c.train.weight_decay) == (3e-4, (0.9, 0.95), 1e-8, 0.1)
    assert (c.train.warmup_steps, c.train.min_lr_ratio, c.train.grad_clip, c.train.seed) == (100, 0.1, 1.0, 1234)
    assert c.parallel.pp_schedule == "1f1b" and c.parallel.init_timeout_s == 1800
    assert c.offload.min_numel == 1 << 18 and c.offload.pipeline_chunks == 4
    assert c.quant.exclude == ("lm_head", "gate", "router", "tok_emb")
    assert "train" in c.to_dict() and c.to_dict()["parallel"]["dp_shard"] == 1


def test_state_dict_keys():
    m = fm.GPT(fm.GPTConfig(vocab_size=64, dim=32, n_layers=1, n_heads=2, n_kv_heads=1, max_seq=16, tie_embeddings=True))
    keys = set(m.state_dict())
    assert {"tok_emb.weight", "norm.weight", "lm_head.weight", "layers.0.attn_norm.weight", "layers.0.ffn_norm.weight",
            "layers.0.attn.wq.weight", "layers.0.attn.wk.weight", "layers.0.attn.wv.weight", "layers.0.attn.wo.weight",
            "layers.0.ffn.w1.weight", "layers.0.ffn.w3.weight", "layers.0.ffn.w2.weight"} == keys
    assert m.lm_head.weight.data_ptr() == m.tok_emb.weight.data_ptr()
    moe = fm.GPT(fm.GPTConfig(vocab_size=64, dim=32, n_layers=1, n_heads=2, n_kv_heads=1, max_seq=16, n_experts=4,
                              n_shared_experts=1))
    mk = set(moe.state_dict())
    assert {"layers.0.ffn.router.gate.weight", "layers.0.ffn.experts.w1", "layers.0.ffn.experts.w3",
            "layers.0.ffn.experts.w2", "layers.0.ffn.shared.w1.weight"} <= mk
    assert moe.state_dict()["layers.0.ffn.experts.w1"].shape == (4, 32, moe.layers["0"].ffn.hidden)


def test_lr_schedule():
    cfg = fm.ForgeConfig()
    cfg.train.__dict__.update(max_steps=1000, warmup_steps=100, lr=1.0, min_lr_ratio=0.1, resume=False, prefetch=False,
                              bf16=False)
    mc = fm.GPTConfig(vocab_size=64, dim=32, n_layers=1, n_heads=2, n_kv_heads=1, max_seq=16)
    tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(64, 16, n=64), micro_batch=4)
    assert tr.lr_at(0) == pytest.approx(0.01)
    assert tr.lr_at(99) == pytest.approx(1.0)
    assert tr.lr_at(100) == pytest.approx(1.0)
    assert tr.lr_at(1000) == pytest.approx(0.1)
    assert tr.lr_at(550) == pytest.approx(0.1 + 0.9 * 0.5)
    tr.close()
