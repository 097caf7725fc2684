"""int8 / fp8 tensor-core products and their quantisers against plain PyTorch statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _C():
    from forgeminds_b200 import ops
    return ops.require()


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


def test_int8_row_quantiser_matches_statement():
    from forgeminds_b200.quant import quantize_rows_int8
    x = _rand((300, 512), 0, 3.0)
    q, s = _C().quant_rows(x, 0, 0)
    want_q, want_s = quantize_rows_int8(x)
    assert torch.allclose(s, want_s, rtol=1e-6, atol=0)
    diff = (q.view(torch.int8).int() - want_q.int()).abs()
    assert diff.max() <= 1 and (diff > 0).float().mean() < 1e-3        # 1/s vs division: rare off-by-one at .5


@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (200, 136, 272), (1024, 1024, 2048)])
def test_int8_gemm_is_exact(M, N, K, cuda_status):
    C = _C()
    a, b = _rand((M, K), 1), _rand((N, K), 2)
    aq, sa = C.quant_rows(a, 0, 0)
    bq, sb = C.quant_rows(b, 0, 0)
    got = C.gemm8(aq, bq, sa, sb, 0, True, cuda_status)
    acc = aq.view(torch.int8).double() @ bq.view(torch.int8).double().T
    want = (acc * sa.double()[:, None] * sb.double()[None, :]).float()
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5), (got - want).abs().max()
    # and it approximates the bf16 product
    ref = a.float() @ b.float().T
    assert (got - ref).norm() / ref.norm() < 0.03


@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (200, 136, 272)])
def test_fp8_gemm_row_scales(M, N, K, cuda_status):
    C = _C()
    a, b = _rand((M, K), 3), _rand((N, K), 4)
    aq, sa = C.quant_rows(a, 1, 0)
    bq, sb = C.quant_rows(b, 1, 0)
    got = C.gemm8(aq, bq, sa, sb, 1, True, cuda_status)
    af = aq.view(torch.float8_e4m3fn).float() * sa[:, None]
    bf = bq.view(torch.float8_e4m3fn).float() * sb[:, None]
    want = af @ bf.T
    assert torch.allclose(got, want, rtol=2e-3, atol=2e-3 * want.abs().max().item()), (got - want).abs().max()
    ref = a.float() @ b.float().T
    assert (got - ref).norm() / ref.norm() < 0.06


@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (200, 136, 400), (512, 1024, 1024)])
def test_fp8_gemm_block_scales(M, N, K, cuda_status):
    from forgeminds_b200.quant import _dequant_fp8
    C = _C()
    a = _rand((M, K), 5) * torch.linspace(0.1, 4.0, K, device="cuda").to(torch.bfloat16)     # scales vary along K
    b = _rand((N, K), 6)
    aq, sa = C.quant_rows(a, 1, 128)
    bq, sb = C.quant_tiles_fp8(b)
    assert sa.shape == (M, (K + 127) // 128) and sb.shape == ((N + 127) // 128, (K + 127) // 128)
    got = C.gemm8(aq, bq, sa, sb, 1, True, cuda_status)
    want = _dequant_fp8(aq.view(torch.float8_e4m3fn), sa, 1, 128) @ _dequant_fp8(bq.view(torch.float8_e4m3fn), sb, 128, 128).T
    assert torch.allclose(got, want, rtol=2e-3, atol=2e-3 * want.abs().max().item()), (got - want).abs().max()
    ref = a.float() @ b.float().T
    assert (got - ref).norm() / ref.norm() < 0.06


@pytest.mark.parametrize("mode", ["int8", "fp8"])
def test_quant_linear_forward_backward(mode, cuda_status):
    from forgeminds_b200.quant import Fp8Linear, Int8Linear
    torch.manual_seed(0)
    lin = torch.nn.Linear(512, 384, bias=False).cuda()
    q = (Int8Linear if mode == "int8" else Fp8Linear).from_linear(lin)
    x = _rand((4, 64, 512), 7).requires_grad_()
    xr = x.detach().clone().requires_grad_()
    y = q(x)
    yr = torch.nn.functional.linear(xr.float(), lin.weight.float())
    assert (y.float() - yr).norm() / yr.norm() < 0.06
    g = _rand(y.shape, 8)
    y.backward(g)
    wq_grad = lin.weight.grad.clone()
    lin.weight.grad = None
    yr.backward(g.float())
    assert (x.grad.float() - xr.grad.float()).norm() / xr.grad.float().norm() < 0.08
    assert (wq_grad.float() - lin.weight.grad.float()).norm() / lin.weight.grad.float().norm() < 0.02


@pytest.mark.parametrize("mode", ["int8", "fp8"])
def test_fused_quantised_projection_equals_separate_ones(mode, cuda_status):
    """q|k|v as one 8-bit product: same outputs and gradients as three quantised linears (row scales are per
    output row, so concatenating the weights changes nothing for int8; fp8 tiles are 128 rows tall and the
    widths here are multiples of 128)."""
    from forgeminds_b200.ops.quant import qlinear_multi
    from forgeminds_b200.quant import Fp8Linear, Int8Linear
    torch.manual_seed(0)
    cls = Int8Linear if mode == "int8" else Fp8Linear
    lins = [torch.nn.Linear(512, n, bias=False).cuda() for n in (256, 128, 128)]
    x = _rand((2, 128, 512), 3).requires_grad_()
    xr = x.detach().clone().requires_grad_()
    y = qlinear_multi(x, tuple(l.weight for l in lins), mode, 128)
    want = torch.cat([cls.from_linear(l)(xr) for l in lins], dim=-1)
    # int8: identical integer products. fp8: the fused form quantises the bf16 copy of the weights, the modules
    # the fp32 weights; a handful of e4m3 codes (3 mantissa bits) round the other way
    assert (y.float() - want.float()).norm() / want.float().norm() < (5e-3 if mode == "int8" else 2e-2)
    g = _rand(y.shape, 4)
    y.backward(g)
    fused_grads = [l.weight.grad.clone() for l in lins]
    for l in lins:
        l.weight.grad = None
    want.backward(g)
    assert (x.grad.float() - xr.grad.float()).norm() / xr.grad.float().norm() < 2e-2
    for a, l in zip(fused_grads, lins):
        assert (a.float() - l.weight.grad.float()).norm() / l.weight.grad.float().norm() < 5e-3      # bf16 products both


@pytest.mark.parametrize("mode", ["int8", "fp8"])
def test_trainer_trains_with_quantised_blocks_on_the_native_engine(mode, cuda_status):
    """quant.mode routes every block projection through the 8-bit GEMMs, also on the flat-store engine."""
    import forgeminds_b200 as fm
    from forgeminds_b200 import ops
    cfg = fm.ForgeConfig()
    cfg.quant.mode = mode
    cfg.train.__dict__.update(max_steps=25, grad_accum=1, lr=3e-3, warmup_steps=5, bf16=True, resume=False,
                              log_every=1000, prefetch=False)
    mc = fm.GPTConfig(vocab_size=512, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=128, ffn_hidden=512)
    tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(512, 128, n=512), micro_batch=4)
    assert tr.store is not None and tr.quant.swapped > 0
    calls = {"n": 0}
    C = ops.require()
    real = C.gemm8

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    C.gemm8 = counting
    try:
        hist = tr.fit()
    finally:
        C.gemm8 = real
        tr.close()
    assert calls["n"] >= 25 * 2 * 8           # four products per block (q|k|v, wo, gate|up, w2), forward + input gradient
    assert hist[-1]["loss"] < 0.75 * hist[0]["loss"], [h["loss"] for h in hist]
