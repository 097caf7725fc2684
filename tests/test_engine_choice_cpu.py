"""Which engine a configuration gets and why (host logic only: no device work here)."""
import types

import pytest
import torch

import forgeminds_b200 as fm
from forgeminds_b200.engine import flat_store_blockers, resident_bytes


def _model():
    return fm.GPT(fm.GPTConfig(vocab_size=64, dim=32, n_layers=2, n_heads=2, n_kv_heads=1, max_seq=16))


def test_every_switch_that_leaves_the_flat_store_gives_its_reason():
    model = _model()
    assert flat_store_blockers(fm.ForgeConfig(), model) == []
    for change, needle in (
            (lambda c: setattr(c.offload, "optimizer", True), "offload.optimizer"),
            (lambda c: setattr(c.quant, "optimizer_8bit", True), "optimizer_8bit"),
            (lambda c: setattr(c.parallel, "fsdp_cpu_offload", True), "fsdp_cpu_offload"),
            (lambda c: setattr(c.train, "compile", True), "train.compile"),
            (lambda c: setattr(c.quant, "mode", "int8_wo"), "int8_wo")):
        cfg = fm.ForgeConfig()
        change(cfg)
        why = flat_store_blockers(cfg, model)
        assert len(why) == 1 and needle in why[0], why
    for mode in ("fp8", "int8"):                      # 8-bit GEMMs of this library stay on the flat store
        cfg = fm.ForgeConfig()
        cfg.quant.mode = mode
        assert flat_store_blockers(cfg, model) == []
    cfg = fm.ForgeConfig()                            # activation offload works on both engines
    cfg.offload.activations = True
    assert flat_store_blockers(cfg, model) == []
    cfg = fm.ForgeConfig()
    cfg.parallel.tp = 2
    model._fm_tp = "dtensor"                          # what apply_tp leaves when the fused kernels cannot serve the mesh
    assert any("DTensor" in w for w in flat_store_blockers(cfg, model))
    model._fm_tp = object()
    assert flat_store_blockers(cfg, model) == []
    cfg = fm.ForgeConfig()
    cfg.parallel.ep = 2
    assert any("expert parallelism" in w for w in flat_store_blockers(cfg, model))      # no fused dispatch attached
    assert flat_store_blockers(cfg, model, kernels=False) == []                         # the CPU form of the engine


def test_resident_bytes_follow_the_flat_store_layout():
    model = _model()
    n = sum(p.numel() for p in model.parameters())
    cfg = fm.ForgeConfig()
    ctx = types.SimpleNamespace(dp_world=8)
    cfg.parallel.dp_shard = 8                         # moments shared by the 8 ranks of the shard group
    assert resident_bytes(model, cfg, ctx) == int(n * (10 + 8 / 8))
    cfg.parallel.dp_shard, cfg.parallel.dp_replicate = 1, 8      # replicas only: the peer step still shards the moments
    assert resident_bytes(model, cfg, ctx) == int(n * (10 + 8 / 8))
    cfg.parallel.dp_shard, cfg.parallel.dp_replicate = 4, 2      # hybrid: shared inside a replica
    assert resident_bytes(model, cfg, ctx) == int(n * (10 + 8 / 4))
    cfg.parallel.fused_comm = False                   # all_reduce path: every rank keeps whole moments
    assert resident_bytes(model, cfg, ctx) == n * 18


def test_engine_switch_is_read_from_the_environment(monkeypatch):
    def trainer():
        cfg = fm.ForgeConfig()
        cfg.train.bf16, cfg.train.max_steps, cfg.train.log_every = False, 1, 100
        mc = fm.GPTConfig(vocab_size=64, dim=32, n_layers=1, n_heads=2, n_kv_heads=1, max_seq=16)
        return fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(64, 16, n=16), micro_batch=2)
    monkeypatch.delenv("FORGEMINDS_FLAT_ENGINE", raising=False)
    t = trainer()
    assert t.eng.name == "library" and t.store is None          # a CPU run: PyTorch engine
    t.close()
    monkeypatch.setenv("FORGEMINDS_FLAT_ENGINE", "1")
    t = trainer()
    assert t.eng.name == "native" and t.store is not None       # the flat store forced on for its bookkeeping
    t.train_step()
    t.close()
