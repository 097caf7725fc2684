"""tcgen05 flash attention (forward + backward, GQA) against an fp32 PyTorch reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, causal):
    # q [B,T,Hq,hd], k/v [B,T,Hkv,hd] -> fp32 attention with grouped heads (one batch entry at a time: the
    # score matrix of the long cases is large)
    if q.shape[0] > 1:
        parts = [_ref(q[i:i + 1], k[i:i + 1], v[i:i + 1], causal) for i in range(q.shape[0])]
        return torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts])
    B, T, Hq, hd = q.shape
    G = Hq // k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(hd)
    if causal:
        mask = torch.ones(T, T, device=q.device, dtype=torch.bool).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    return (p @ vf).permute(0, 2, 1, 3), torch.logsumexp(s, -1)


def _qkv(B, T, Hq, Hkv, hd, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(B, T, (Hq + 2 * Hkv) * hd, device="cuda", generator=g)).to(torch.bfloat16)


CASES = [
    (2, 256, 4, 2, 64, True),
    (1, 512, 8, 2, 64, True),
    (2, 384, 4, 4, 128, True),
    (1, 256, 4, 1, 80, True),
    (1, 256, 2, 2, 32, True),
    (2, 256, 4, 2, 64, False),
    (1, 200, 4, 2, 64, True),      # sequence not a multiple of the tile
    (4, 2048, 16, 4, 64, True),    # the benchmark shape: 16 kv tiles, groups of four query heads
    (1, 2048, 8, 2, 128, True),
    (1, 1100, 8, 2, 80, True),     # head dim 80, ragged last tile (the dQ boxes are clipped at T)
]


@pytest.mark.parametrize("B,T,Hq,Hkv,hd,causal", CASES)
def test_forward(B, T, Hq, Hkv, hd, causal, cuda_status):
    from forgeminds_b200 import ops
    C = ops.require()
    qkv = _qkv(B, T, Hq, Hkv, hd, 1)
    q = qkv[..., : Hq * hd].unflatten(-1, (Hq, hd))
    k = qkv[..., Hq * hd: (Hq + Hkv) * hd].unflatten(-1, (Hkv, hd))
    v = qkv[..., (Hq + Hkv) * hd:].unflatten(-1, (Hkv, hd))
    o, lse = C.attn_fwd(q, k, v, 1.0 / math.sqrt(hd), causal, cuda_status)
    ro, rl = _ref(q, k, v, causal)
    assert (o.float() - ro).abs().max() < 0.03, (o.float() - ro).abs().max()
    assert (lse - rl).abs().max() < 0.02


@pytest.mark.parametrize("B,T,Hq,Hkv,hd,causal", CASES)
def test_backward(B, T, Hq, Hkv, hd, causal, cuda_status):
    from forgeminds_b200.ops import functional as Fn
    qkv = _qkv(B, T, Hq, Hkv, hd, 2).requires_grad_()
    out = Fn.attention_qkv(qkv, Hq, Hkv, hd, causal)
    g = torch.randn_like(out)
    out.backward(g)
    ref_in = qkv.detach().float().requires_grad_()
    q = ref_in[..., : Hq * hd].unflatten(-1, (Hq, hd))
    k = ref_in[..., Hq * hd: (Hq + Hkv) * hd].unflatten(-1, (Hkv, hd))
    v = ref_in[..., (Hq + Hkv) * hd:].unflatten(-1, (Hkv, hd))
    ro, _ = _ref(q, k, v, causal)
    ro.reshape(B, T, Hq * hd).backward(g.float())
    got, want = qkv.grad.float(), ref_in.grad
    for name, lo, hi in (("dq", 0, Hq * hd), ("dk", Hq * hd, (Hq + Hkv) * hd), ("dv", (Hq + Hkv) * hd, None)):
        a, b = got[..., lo:hi], want[..., lo:hi]
        rel = (a - b).norm() / b.norm().clamp(min=1e-6)
        assert rel < 2.5e-2, f"{name}: relative error {rel}"


@pytest.mark.parametrize("B,T,Hq,Hkv,hd", [(2, 256, 4, 2, 64), (1, 1100, 8, 2, 80), (1, 512, 8, 2, 128)])
def test_rope_folded_into_attention(B, T, Hq, Hkv, hd, cuda_status):
    """RoPE applied inside the attention node (backward rotation reads the fp32 dQ sum) against the
    separate rotate-then-attend nodes and against fp32 autograd."""
    from forgeminds_b200.models.gpt import rope_tables
    from forgeminds_b200.ops import functional as Fn
    cos, sin = rope_tables(T, hd, 10000.0, "cuda", torch.float32)
    cos, sin = cos.reshape(T, hd // 2).contiguous(), sin.reshape(T, hd // 2).contiguous()
    raw = _qkv(B, T, Hq, Hkv, hd, 3)
    g = torch.randn(B, T, Hq * hd, device="cuda", dtype=torch.bfloat16)
    grads = []
    for folded in (True, False):
        leaf = raw.clone().requires_grad_()
        x = leaf * 1.0                                  # a non-leaf buffer the node may rotate in place
        if folded:
            out = Fn.attention_qkv(x, Hq, Hkv, hd, True, rope=(cos, sin))
        else:
            out = Fn.attention_qkv(Fn.rope_qkv_(x, cos, sin, Hq, Hkv, hd), Hq, Hkv, hd, True)
        out.backward(g)
        grads.append((out.detach().float(), leaf.grad.float()))
    assert torch.equal(grads[0][0], grads[1][0])
    rel = (grads[0][1] - grads[1][1]).norm() / grads[1][1].norm()
    assert rel < 1e-2, rel

    # fp32 reference of rotate + attend
    ref_in = raw.float().requires_grad_()
    n_rot = Hq + Hkv
    heads = ref_in.unflatten(-1, (Hq + 2 * Hkv, hd))
    a, b = heads[..., : hd // 2], heads[..., hd // 2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    rot = torch.cat([a * c - b * s, a * s + b * c], -1)
    heads = torch.cat([rot[:, :, :n_rot], heads[:, :, n_rot:]], 2)
    ro, _ = _ref(heads[:, :, :Hq], heads[:, :, Hq:n_rot], heads[:, :, n_rot:], True)
    ro.reshape(B, T, Hq * hd).backward(g.float())
    rel = (grads[0][1] - ref_in.grad).norm() / ref_in.grad.norm()
    assert rel < 2.5e-2, rel
