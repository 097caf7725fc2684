"""Flat parameter store + fused AdamW (PyTorch statement of the kernel on CPU) against torch.optim.AdamW."""
import torch

import forgeminds_b200 as fm
from forgeminds_b200.parallel.flat import FlatAdamW, FlatParamStore


def _gpt():
    torch.manual_seed(0)
    return fm.GPT(fm.GPTConfig(vocab_size=128, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=16, native=False))


def test_parameters_become_views_and_fused_projections_are_adjacent():
    from forgeminds_b200.ops.functional import _adjacent
    m = _gpt()
    before = {k: v.clone() for k, v in m.state_dict().items()}
    store = FlatParamStore(m, "cpu")
    for k, v in m.state_dict().items():
        assert torch.equal(v, before[k]), k
    blk = m.layers["0"]
    shadows = [p._fm_shadow[0] for p in (blk.attn.wq.weight, blk.attn.wk.weight, blk.attn.wv.weight)]
    assert _adjacent(shadows)
    assert _adjacent([blk.ffn.w1.weight._fm_main_grad, blk.ffn.w3.weight._fm_main_grad])
    assert [b.name for b in store.buckets] == ["block0", "block1", "rest"]
    assert all(p.grad is not None and p.grad.data_ptr() == p._fm_main_grad.data_ptr() for p in store.params)
    assert torch.equal(store.shadow.float(), store.master.bfloat16().float())


def test_fused_adamw_matches_torch_adamw():
    a, b = _gpt(), _gpt()
    store = FlatParamStore(b, "cpu")
    opt_b = FlatAdamW(store, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    decay = [p for p in a.parameters() if p.ndim >= 2]
    rest = [p for p in a.parameters() if p.ndim < 2]
    opt_a = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}],
                              lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    tok = torch.randint(0, 128, (2, 16))
    for _ in range(3):
        la, _ = a(tok, labels=tok)
        lb, _ = b(tok, labels=tok)
        la.backward()
        lb.backward()
        opt_a.step()
        opt_a.zero_grad()
        opt_b.step()
        opt_b.zero_grad()
    for (n, pa), pb in zip(a.named_parameters(), b.parameters()):
        assert torch.allclose(pa, pb, atol=2e-6), n
    assert torch.equal(store.shadow[: 64 * 128].float(), store.master[: 64 * 128].bfloat16().float())


def test_skip_flag_and_clip_coefficient_live_on_the_device():
    m = _gpt()
    store = FlatParamStore(m, "cpu")
    opt = FlatAdamW(store, lr=1e-2)
    tok = torch.randint(0, 128, (2, 16))
    m(tok, labels=tok)[0].backward()
    before = store.master.clone()
    opt.ctl[1] = 0.0
    opt.step()
    assert torch.equal(store.master, before)
    opt.ctl[1] = 1.0
    opt.step()
    assert not torch.equal(store.master, before)
    out = torch.zeros(1)
    store.grad_sq_norm(out)
    assert torch.allclose(out[0], sum(p.grad.float().pow(2).sum() for p in m.parameters()), rtol=1e-5)


def test_state_dict_roundtrip_keeps_the_flat_layout():
    m = _gpt()
    store = FlatParamStore(m, "cpu")
    opt = FlatAdamW(store, lr=1e-2)
    tok = torch.randint(0, 128, (2, 16))
    m(tok, labels=tok)[0].backward()
    opt.step()
    sd = opt.state_dict()
    m2 = _gpt()
    store2 = FlatParamStore(m2, "cpu")
    opt2 = FlatAdamW(store2, lr=1e-2)
    opt2.load_state_dict(sd)
    assert torch.equal(opt2.exp_avg, opt.exp_avg) and opt2.steps == 1
    p = store2.params[0]
    assert opt2.state[p]["exp_avg"].data_ptr() == opt2.exp_avg[store2._offset[p]:].data_ptr()
