"""Degenerate inputs: empty and fully ignored label sets, odd sequence lengths, more ranks than samples,
width-one rows, mismatched shapes, and the Forge conventions for losses that are not plain scalars."""
import math

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import forgeminds_b200 as fm
from forgeminds_b200 import kernels as K
from forgeminds_b200.loss import chunked_cross_entropy, logits_cross_entropy


# ------------------------------------------------------------------ losses
def test_cross_entropy_with_every_label_ignored_is_zero_and_differentiable():
    h = torch.randn(6, 8, requires_grad=True)
    w = torch.randn(11, 8, requires_grad=True)
    loss = chunked_cross_entropy(h, w, torch.full((6,), -100), chunk=4)
    assert loss.item() == 0.0
    loss.backward()
    assert torch.count_nonzero(h.grad) == 0 and torch.count_nonzero(w.grad) == 0


def test_cross_entropy_of_no_tokens():
    h = torch.zeros(0, 8, requires_grad=True)
    w = torch.randn(11, 8, requires_grad=True)
    loss = chunked_cross_entropy(h, w, torch.zeros(0, dtype=torch.long))
    assert loss.item() == 0.0 and loss.requires_grad
    assert logits_cross_entropy(torch.zeros(0, 11), torch.zeros(0, dtype=torch.long)).item() == 0.0


@pytest.mark.parametrize("chunk", [1, 5, 64])
def test_chunked_cross_entropy_equals_the_plain_one(chunk):
    torch.manual_seed(0)
    h = torch.randn(3, 7, 8, requires_grad=True)
    w = torch.randn(13, 8, requires_grad=True)
    y = torch.randint(0, 13, (3, 7))
    y[0, :3] = -100
    want = F.cross_entropy(F.linear(h, w).reshape(-1, 13), y.reshape(-1), ignore_index=-100)
    got = chunked_cross_entropy(h, w, y, chunk=chunk)
    assert torch.allclose(got, want, atol=1e-6)
    gw, = torch.autograd.grad(got, w, retain_graph=True)
    ww, = torch.autograd.grad(want, w)
    assert torch.allclose(gw, ww, atol=1e-6)
    assert torch.allclose(logits_cross_entropy(F.linear(h, w), y, chunk=chunk), want, atol=1e-6)


# ------------------------------------------------------------------ data
@pytest.mark.parametrize("seq", [1, 7, 8, 13])
def test_synthetic_corpus_handles_any_sequence_length(seq):
    ds = fm.SyntheticLM(50, seq, n=5)
    item = ds[4]
    assert item["input_ids"].shape == (seq,) and item["labels"].shape == (seq,)
    assert torch.equal(item["input_ids"][1:], item["labels"][:-1])


def test_token_file_shorter_than_two_windows(tmp_path):
    path = tmp_path / "tok.bin"
    np.arange(10, dtype=np.uint16).tofile(path)
    ds = fm.TokenFile(str(path), seq=4)
    assert len(ds) == 2
    assert ds[1]["input_ids"].tolist() == [4, 5, 6, 7] and ds[1]["labels"].tolist() == [5, 6, 7, 8]
    empty = tmp_path / "few.bin"
    np.arange(3, dtype=np.uint16).tofile(empty)
    assert len(fm.TokenFile(str(empty), seq=4)) == 0


def test_sampler_with_more_ranks_than_samples_yields_nothing():
    s = fm.ResumableSampler(3, dp_rank=2, dp_world=8, seed=0)
    assert list(s) == [] and len(s) == 0


def test_sampler_skip_beyond_the_epoch_is_harmless():
    s = fm.ResumableSampler(16, dp_rank=0, dp_world=2, seed=0)
    s.skip = 100
    assert list(s) == [] and len(s) >= 0
    assert len(list(s)) == 8                               # the skip applied to one pass only


def test_batch_stream_over_nothing_says_so():
    ctx = fm.init_distributed(fm.ParallelConfig())
    dl, sampler = fm.build_loader(fm.SyntheticLM(50, 8, n=2), 4, ctx, seed=0)       # 2 samples, batch of 4, drop_last
    with pytest.raises((RuntimeError, ValueError)) as err:
        stream = fm.BatchStream(dl, sampler, ctx.device, threaded=False)
        stream.next()
    assert "batch" in str(err.value).lower() or "empty" in str(err.value).lower()


# ------------------------------------------------------------------ kernels API on odd shapes
def test_rms_norm_on_strided_input_and_zero_rows():
    x = torch.randn(4, 6, 10)[:, ::2, :].transpose(0, 1)
    w = torch.rand(10) + 0.5
    assert not x.is_contiguous()
    assert torch.allclose(K.rms_norm(x, w, 1e-6), F.rms_norm(x, (10,), w, 1e-6), atol=1e-6)
    none = torch.zeros(0, 10)
    assert K.rms_norm(none, w, 1e-6).shape == (0, 10)
    zero = torch.zeros(3, 10)
    assert torch.isfinite(K.rms_norm(zero, w, 1e-6)).all()


def test_rms_norm_of_width_one():
    x = torch.tensor([[2.0], [-3.0], [0.0]], requires_grad=True)
    y = K.rms_norm(x, torch.ones(1), 1e-6)
    assert torch.allclose(y.detach(), torch.tensor([[1.0], [-1.0], [0.0]]), atol=1e-3)
    y.sum().backward()
    assert torch.isfinite(x.grad).all()


def test_kl_over_a_single_class_is_zero():
    s, t = torch.randn(5, 1, requires_grad=True), torch.randn(5, 1)
    kl = K.kl_div(s, t)
    assert abs(float(kl)) < 1e-7
    kl.backward()
    assert torch.count_nonzero(s.grad) == 0


def test_swiglu_split_with_one_hidden_unit():
    gu = torch.tensor([[1.0, 2.0], [-1.0, 0.5]])
    want = F.silu(gu[:, :1]) * gu[:, 1:]
    assert torch.allclose(K.swiglu_split(gu), want, atol=1e-6)
    with pytest.raises((ValueError, RuntimeError)):
        K.swiglu_split(torch.randn(2, 3))                 # odd width cannot be halved


def test_swiglu_refuses_shapes_that_would_broadcast():
    with pytest.raises((ValueError, RuntimeError)):
        K.swiglu(torch.randn(4, 8), torch.randn(1, 8))
    with pytest.raises((ValueError, RuntimeError)):
        K.swiglu(torch.randn(4, 8), torch.randn(4, 1))


# ------------------------------------------------------------------ Forge conventions
def _tiny_forge(model, **kw):
    kw.setdefault("precision", "fp32")
    kw.setdefault("quiet", True)
    kw.setdefault("async_batches", False)
    return fm.Forge(model, torch.optim.SGD(model.parameters(), lr=0.1), **kw)


def test_forge_takes_the_loss_entry_of_a_dict():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(4, 1)

        def forward(self, x):
            return {"loss": self.lin(x).pow(2).mean(), "logits": self.lin(x)}
    st = _tiny_forge(Net()).step(torch.randn(3, 4))
    assert st.step == 1 and math.isfinite(st.loss)


def test_forge_without_clipping_reports_nan_norm_and_still_updates():
    model = nn.Linear(4, 1)
    before = model.weight.detach().clone()
    st = _tiny_forge(model, clip=0, loss_fn=lambda out, b: out.pow(2).mean()).step(torch.randn(3, 4))
    assert math.isnan(st.grad_norm) and not st.skipped
    assert not torch.equal(before, model.weight.detach())


def test_forge_averages_a_loss_that_is_not_a_scalar():
    model = nn.Linear(4, 2)
    st = _tiny_forge(model, loss_fn=lambda out, b: out.pow(2)).step(torch.randn(5, 4))       # [5, 2] "loss"
    assert math.isfinite(st.loss) and st.step == 1


def test_forge_refuses_an_output_without_a_loss():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(4, 1)

        def forward(self, x):
            return "not a loss"
    with pytest.raises(TypeError, match="loss"):
        _tiny_forge(Net()).step(torch.randn(3, 4))
