"""OffloadedAdamW against torch.optim.AdamW, activation offload hooks, pinned pool."""
import pytest
import torch
import torch.nn as nn

from forgeminds_b200.config import OffloadConfig
from forgeminds_b200.offload import ActivationOffload, OffloadedAdamW, apply_activation_offload
from forgeminds_b200.perf import pinned_pool


def _pair():
    torch.manual_seed(0)
    a = nn.Sequential(nn.Linear(6, 12), nn.GELU(), nn.Linear(12, 3))
    b = nn.Sequential(nn.Linear(6, 12), nn.GELU(), nn.Linear(12, 3))
    b.load_state_dict(a.state_dict())
    return a, b


@pytest.mark.parametrize("accum", [1, 2, 3])
@pytest.mark.parametrize("chunks", [1, 4])
def test_matches_adamw(accum, chunks):
    a, b = _pair()
    ref = torch.optim.AdamW(a.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    cfg = OffloadConfig(smart=False, pipeline_chunks=chunks)
    off = OffloadedAdamW([{"params": list(b.parameters()), "weight_decay": 0.1}], 1e-2, (0.9, 0.95), 1e-8, cfg)
    g = torch.Generator().manual_seed(1)
    for _ in range(3):
        for _ in range(accum):
            x = torch.randn(5, 6, generator=g)
            (a(x).pow(2).mean() / accum).backward()
            (b(x).pow(2).mean() / accum).backward()
        ref.step()
        ref.zero_grad()
        off.step()
        off.zero_grad()
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert torch.allclose(pa, pb, atol=1e-6)
    rep = off.report()
    assert rep["params"] == 4 and rep["chunks"] == chunks


def test_host_clip_equals_torch_clip():
    a, b = _pair()
    off = OffloadedAdamW([{"params": list(b.parameters())}], 1e-2, cfg=OffloadConfig(smart=False))
    x = torch.randn(4, 6)
    a(x).sum().backward()
    b(x).sum().backward()
    want = torch.nn.utils.clip_grad_norm_(a.parameters(), 0.5)
    got = off.clip_grad_norm_(0.5)
    assert torch.allclose(want, got, atol=1e-6)
    clipped = torch.stack([g.norm() for g in off._accs]).norm()
    assert clipped <= 0.5 + 1e-5


def test_smart_policy_keeps_small_tensors_and_state_roundtrip():
    _, b = _pair()
    off = OffloadedAdamW([{"params": list(b.parameters())}], 1e-2, cfg=OffloadConfig(smart=True, min_numel=50))
    b(torch.randn(2, 6)).sum().backward()
    assert b[0].weight.grad is None and b[2].bias.grad is not None       # 72 elements moved, 3 stayed
    off.step()
    sd = off.state_dict()
    _, c = _pair()
    off2 = OffloadedAdamW([{"params": list(c.parameters())}], 1e-2, cfg=OffloadConfig(smart=False))
    off2.load_state_dict(sd)
    for pb, pc in zip(b.parameters(), c.parameters()):
        assert torch.equal(pb, pc)
    assert "OffloadedAdamW" in repr(off)


def test_activation_offload_is_transparent_on_cpu():
    class Tiny(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleDict({"0": nn.Linear(8, 8), "1": nn.Linear(8, 8)})

        def forward(self, x):
            for l in self.layers.values():
                x = torch.tanh(l(x))
            return x
    torch.manual_seed(0)
    m = Tiny()
    x = torch.randn(3, 8)
    m(x).sum().backward()
    want = [p.grad.clone() for p in m.parameters()]
    m.zero_grad()
    apply_activation_offload(m, OffloadConfig(act_min_bytes=1, act_layers=0.5))
    m(x).sum().backward()
    for p, g in zip(m.parameters(), want):
        assert torch.allclose(p.grad, g)
    with ActivationOffload(1):
        y = (torch.randn(4, 4, requires_grad=True) * 2).sum()
    y.backward()


def test_pinned_pool_reuses_buffers():
    pool = pinned_pool(pin=False)
    a = pool.get((4, 4), torch.float32)
    pool.put(a)
    b = pool.get((4, 4), torch.float32)
    assert a.data_ptr() == b.data_ptr() and (pool.hits, pool.misses) == (1, 1)
    pool.clear()
