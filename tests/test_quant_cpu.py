"""Quantised linear layers: the PyTorch emulation of the int8 / block-scaled fp8 kernels."""
import pytest
import torch
import torch.nn as nn

import forgeminds_b200 as fm
from forgeminds_b200.quant import (Fp8Linear, Int8Linear, quantize_blocks_fp8, quantize_model, quantize_rows_int8,
                                   resolve_backend)


def test_quantisers_roundtrip():
    x = torch.randn(37, 200)
    q, s = quantize_rows_int8(x)
    assert q.dtype == torch.int8 and (q.float() * s[:, None] - x).abs().max() <= s.max() * 0.51
    q8, s8 = quantize_blocks_fp8(x, 1, 128)
    assert q8.dtype == torch.float8_e4m3fn and s8.shape == (37, 2)
    qw, sw = quantize_blocks_fp8(torch.randn(130, 260), 128, 128)
    assert sw.shape == (2, 3)


@pytest.mark.parametrize("cls,tol", [(Int8Linear, 0.03), (Fp8Linear, 0.08)])
def test_layers_track_the_fp32_linear(cls, tol):
    torch.manual_seed(0)
    lin = nn.Linear(256, 128, bias=True)
    q = cls.from_linear(lin)
    x = torch.randn(16, 256, requires_grad=True)
    y = q(x)
    ref = lin(x)
    assert (y - ref).norm() / ref.norm() < tol
    y.sum().backward()
    assert q.weight.grad is not None and x.grad is not None
    assert q.weight is lin.weight                                   # the master weight is shared, not copied


def test_quantize_model_respects_exclude_and_backends():
    mc = fm.GPTConfig(vocab_size=64, dim=32, n_layers=1, n_heads=2, n_kv_heads=1, max_seq=16)
    m = fm.GPT(mc)
    st = quantize_model(m, fm.QuantConfig(mode="int8"))
    assert st.backend == "native" and st.swapped == 7
    assert isinstance(m.layers["0"].attn.wq, Int8Linear) and not isinstance(m.lm_head, Int8Linear)
    tok = torch.randint(0, 64, (2, 16))
    loss, _ = m(tok, labels=tok)
    loss.backward()
    assert quantize_model(fm.GPT(mc), fm.QuantConfig()).backend == "none"
    with pytest.raises(RuntimeError):
        resolve_backend(fm.QuantConfig(mode="fp8", backend="te"))
    with pytest.raises(ValueError):
        resolve_backend(fm.QuantConfig(mode="fp4"))
    wo = fm.GPT(mc)
    quantize_model(wo, fm.QuantConfig(mode="int8_wo"))
    assert any(p.requires_grad for p in wo.parameters())
    with st.autocast():
        pass
