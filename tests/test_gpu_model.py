"""The sm_100a block path of GPT against the PyTorch path of the same module (same weights)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _models(**over):
    import forgeminds_b200 as fm
    torch.manual_seed(0)
    base = dict(vocab_size=1024, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=256, ffn_hidden=704)
    base.update(over)
    native = fm.GPT(fm.GPTConfig(native=True, **base)).cuda()
    plain = fm.GPT(fm.GPTConfig(native=False, **base)).cuda()
    plain.load_state_dict(native.state_dict())
    return native, plain


def test_loss_and_grads_match_torch_path(cuda_status):
    native, plain = _models()
    tok = torch.randint(0, 1024, (2, 256), device="cuda")
    lab = torch.randint(0, 1024, (2, 256), device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        ln, _ = native(tok, labels=lab)
        lp, _ = plain(tok, labels=lab)
    ln.backward()
    lp.backward()
    assert abs(ln.item() - lp.item()) < 3e-2, (ln.item(), lp.item())
    for (name, a), (_, b) in zip(native.named_parameters(), plain.named_parameters()):
        ga, gb = a.grad.float(), b.grad.float()
        rel = (ga - gb).norm() / gb.norm().clamp(min=1e-6)
        assert rel < 6e-2, f"{name}: relative gradient error {rel}"


def test_logits_path(cuda_status):
    native, plain = _models(tie_embeddings=True)
    tok = torch.randint(0, 1024, (1, 128), device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16), torch.no_grad():
        a = native(tok).float()
        b = plain(tok).float()
    assert (a - b).abs().max() < 0.15


def test_trainer_native_engine_learns_and_matches_library(tmp_path, cuda_status):
    import forgeminds_b200 as fm
    losses = {}
    for engine in ("native", "library"):
        cfg = fm.ForgeConfig()
        cfg.train.__dict__.update(max_steps=30, grad_accum=2, lr=3e-3, warmup_steps=5, bf16=True, resume=False,
                                  log_every=1000, native=(engine == "native"), prefetch=False)
        mc = fm.GPTConfig(vocab_size=512, dim=128, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=128, ffn_hidden=384)
        ds = fm.SyntheticLM(512, 128, n=512)
        tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, ds, micro_batch=4)
        assert (tr.store is not None) == (engine == "native")
        hist = tr.fit()
        tr.close()
        losses[engine] = [h["loss"] for h in hist]
    assert losses["native"][-1] < 0.6 * losses["native"][0]
    assert abs(losses["native"][0] - losses["library"][0]) < 0.05
    assert abs(losses["native"][-1] - losses["library"][-1]) < 0.35


def test_native_step_has_one_host_sync(cuda_status):
    import forgeminds_b200 as fm
    cfg = fm.ForgeConfig()
    cfg.train.__dict__.update(max_steps=10, grad_accum=2, bf16=True, resume=False, log_every=1000, prefetch=False)
    mc = fm.GPTConfig(vocab_size=512, dim=128, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=128, ffn_hidden=384)
    tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(512, 128, n=256), micro_batch=4)
    tr.train_step()
    with fm.count_host_syncs() as c:
        for _ in range(3):
            tr.train_step()
    tr.close()
    assert c.own <= 3, c.report()


def test_moe_native_matches_torch_path(cuda_status):
    import forgeminds_b200 as fm
    from forgeminds_b200.moe import MoE
    torch.manual_seed(0)
    moe = MoE(256, 512, 8, 2, grouped_mm=True).cuda()
    ref = copy.deepcopy(moe)
    x = (torch.randn(1000, 256, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    xr = x.detach().clone().requires_grad_()
    # the dropless path takes its row buffers uncleared: hand the allocator blocks full of NaN to reuse
    junk = [torch.full((8 << 20,), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(4)]
    del junk
    out = moe(x)                               # bf16 CUDA input -> kernels
    assert moe.last_aux is not None
    with torch.autocast("cuda", dtype=torch.bfloat16):
        want = ref._dispatch_torch(xr, *ref.router(xr)[:2])
        _, _, aux_r, z_r = ref.router(xr)
    assert (out.float() - want.float()).abs().max() < 0.05
    assert abs(moe.last_aux.item() - (ref.aux_coef * aux_r + ref.z_coef * z_r).item()) < 2e-3
    g = torch.randn_like(out)
    junk = [torch.full((8 << 20,), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(4)]
    del junk
    (out.float() * g.float()).sum().backward()
    (want.float() * g.float()).sum().backward()
    assert torch.isfinite(x.grad).all()
    assert (x.grad.float() - xr.grad.float()).norm() / xr.grad.float().norm() < 0.08
    for name in ("w1", "w3", "w2"):
        a, b = getattr(moe.experts, name).grad.float(), getattr(ref.experts, name).grad.float()
        assert torch.isfinite(a).all(), name
        assert (a - b).norm() / b.norm() < 0.08, name


def test_moe_capacity_drops_overflow(cuda_status):
    from forgeminds_b200.moe import MoE
    torch.manual_seed(1)
    moe = MoE(128, 256, 4, 2, grouped_mm=True, capacity_factor=1.0).cuda()
    ref = copy.deepcopy(moe)
    from forgeminds_b200.ops.moe import ALIGN
    ref.capacity = lambda n: (moe.capacity(n) + ALIGN - 1) // ALIGN * ALIGN       # regions are whole row tiles
    x = (torch.randn(2048, 128, device="cuda")).to(torch.bfloat16)
    out = moe(x)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        w, idx, _, _ = ref.router(x)
        want = ref._dispatch_torch(x, w, idx)
    assert (out.float() - want.float()).abs().max() < 0.06
