"""One host synchronisation per optimizer step (reads of CPU tensors are counted here on purpose)."""
import torch

import forgeminds_b200 as fm


def _trainer(**over):
    cfg = fm.ForgeConfig()
    cfg.train.__dict__.update(max_steps=100, bf16=False, log_every=1000, resume=False, prefetch=False)
    cfg.train.__dict__.update({k: v for k, v in over.items() if hasattr(cfg.train, k)})
    if over.get("offload"):
        cfg.offload.optimizer, cfg.offload.smart = True, False
    mc = fm.GPTConfig(vocab_size=128, dim=32, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=16,
                      n_experts=over.get("experts", 0))
    ds = fm.SyntheticLM(128, 16, n=256)
    return fm.Trainer(lambda ctx: fm.GPT(mc, fm.moe_kwargs(ctx, cfg) if over.get("experts") else None), cfg, ds,
                      micro_batch=4)


def _own_syncs(tr, steps=3):
    tr.train_step()
    with fm.count_host_syncs(count_cpu=True) as c:
        for _ in range(steps):
            tr.train_step()
    tr.close()
    return c


def test_dense_accum_spike_ac():
    for kw in ({}, {"grad_accum": 3}, {"skip_spike_factor": 3.0}, {"ac": "full"}, {"ac": "selective"}):
        c = _own_syncs(_trainer(**kw))
        assert c.own <= 3, (kw, c.report())


def test_moe_budget():
    c = _own_syncs(_trainer(experts=4))
    assert c.own <= 3 * (1 + 2), c.report()      # torch path: one read per MoE layer for the split sizes


def test_counter_is_removed_after_use():
    orig = torch.Tensor.item
    with fm.count_host_syncs(count_cpu=True) as c:
        torch.ones(1).item()
        assert torch.Tensor.item is not orig
    assert c.count == 1 and c.external == 1
    assert torch.Tensor.item is orig
    assert fm.host_syncs() >= 1
    assert "host sync" in c.report()
