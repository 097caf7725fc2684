"""Decoder-only transformer: RMSNorm, RoPE (half-split), grouped-query attention, SwiGLU, optional MoE.

Module tree, parameter names, initialisation and the ``forward(tokens, labels) -> (ce, aux)``
contract follow the reference's ``forgemind/models/gpt.py:29-281`` so that state dicts are
interchangeable. What differs is execution: on a B200 with bf16 compute every block runs on the
hand-written kernels of :mod:`forgeminds_b200.ops` -- one fused q|k|v GEMM and one gate|up GEMM on
tcgen05, RoPE applied in place on the fused projection, flash attention reading q/k/v as slices of
that buffer, residual adds in the GEMM epilogues, and the lm_head fused with the cross-entropy.
Everywhere else (CPU, fp32) the same modules run plain PyTorch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..loss import chunked_cross_entropy

__all__ = ["GPTConfig", "GPT", "RMSNorm", "Attention", "SwiGLU", "Block", "rope_tables", "apply_rope",
           "clear_rope_cache"]


@dataclass
class GPTConfig:
    vocab_size: int = 32000
    dim: int = 512
    n_layers: int = 8
    n_heads: int = 8
    n_kv_heads: int = 4
    ffn_mult: float = 8 / 3
    max_seq: int = 2048
    rope_theta: float = 10000.0
    rope_high_precision: bool = False
    tie_embeddings: bool = False
    loss_chunk: int = 4096
    n_experts: int = 0
    top_k: int = 2
    moe_every: int = 1
    n_shared_experts: int = 0
    expert_hidden_mult: float = 1.0
    expert_grouped_mm: bool = True
    aux_coef: float = 1e-2
    z_coef: float = 1e-3
    mixer: str = "attn"                 # "attn" | "cell"
    # ---- additions of this library
    ffn_hidden: Optional[int] = None    # explicit MLP width (overrides ceil64(dim * ffn_mult))
    capacity_factor: float = 0.0        # > 0: experts take at most cf * tokens * top_k / n_experts rows
    native: Optional[bool] = None       # None: sm_100a kernels whenever they can run; False: PyTorch only

    def mlp_hidden(self) -> int:
        if self.ffn_hidden:
            return int(self.ffn_hidden)
        return (int(self.dim * self.ffn_mult) + 63) // 64 * 64


# ------------------------------------------------------------------------------ RoPE tables
_TABLES: dict = {}
_TABLES_MAX = 32


def rope_tables(T: int, hd: int, theta: float, device, dtype):
    """``cos, sin`` of shape ``[1, T, 1, hd/2]``, cached per (64-token length bucket, head_dim,
    theta, device, dtype)."""
    n = max(64, -(-int(T) // 64) * 64)
    device = torch.device(device)
    key = (n, int(hd), float(theta), device.type, device.index, dtype)
    hit = _TABLES.get(key)
    if hit is None:
        if len(_TABLES) >= _TABLES_MAX:
            _TABLES.clear()
        freq = theta ** (-torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd)
        angle = torch.outer(torch.arange(n, device=device, dtype=torch.float32), freq)
        hit = (angle.cos().to(dtype)[None, :, None, :].contiguous(),
               angle.sin().to(dtype)[None, :, None, :].contiguous())
        _TABLES[key] = hit
    return hit[0][:, :T], hit[1][:, :T]


def clear_rope_cache() -> None:
    _TABLES.clear()


def apply_rope(x, cos, sin):
    """Half-split rotation of ``x [B,T,H,hd]``."""
    a, b = x.chunk(2, dim=-1)
    return torch.cat((a * cos - b * sin, a * sin + b * cos), dim=-1)


def _is_quantised(linear) -> bool:
    """True for the int8 / fp8 linear layers that ``quantize_model`` swaps in."""
    return hasattr(linear, "mode") and hasattr(linear, "block") and isinstance(linear, nn.Linear)


def _native_ok(x: torch.Tensor, flag: Optional[bool]) -> bool:
    """Whether this call should run on the sm_100a kernels."""
    if flag is False or not x.is_cuda:
        return False
    bf16 = x.dtype == torch.bfloat16 or (torch.is_autocast_enabled() and
                                         torch.get_autocast_dtype("cuda") == torch.bfloat16)
    if not bf16:
        return False
    from .. import ops
    if ops.available():
        return True
    if flag is True or torch.cuda.get_device_capability(x.device)[0] == 10:
        ops.require()      # a B200 without the extension is a build problem, not a reason to fall back
    return False


# ------------------------------------------------------------------------------ modules
class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight.to(x.dtype), self.eps)


class Attention(nn.Module):
    def __init__(self, c: GPTConfig):
        super().__init__()
        self.hd = c.dim // c.n_heads
        self.theta = c.rope_theta
        self.hp = c.rope_high_precision
        self.register_buffer("_cos", torch.empty(0), persistent=False)
        self.register_buffer("_sin", torch.empty(0), persistent=False)
        self.wq = nn.Linear(c.dim, c.n_heads * self.hd, bias=False)
        self.wk = nn.Linear(c.dim, c.n_kv_heads * self.hd, bias=False)
        self.wv = nn.Linear(c.dim, c.n_kv_heads * self.hd, bias=False)
        self.wo = nn.Linear(c.n_heads * self.hd, c.dim, bias=False)

    def cache_rope(self, device, dtype, seq: int) -> "Attention":
        cos, sin = rope_tables(seq, self.hd, self.theta, device, torch.float32 if self.hp else dtype)
        self._cos, self._sin = cos, sin
        return self

    def _tables(self, x, T):
        stale = self._cos.numel() == 0 or self._cos.shape[1] < T or self._cos.device != x.device or \
            (not self.hp and self._cos.dtype != x.dtype)
        if stale:
            self.cache_rope(x.device, x.dtype, T)
        if self._cos.shape[1] == T:
            return self._cos, self._sin
        return self._cos[:, :T], self._sin[:, :T]

    def forward(self, x):
        B, T, _ = x.shape
        q = self.wq(x).reshape(B, T, -1, self.hd)       # -1: heads held by this rank under tensor parallelism
        k = self.wk(x).reshape(B, T, -1, self.hd)
        v = self.wv(x).reshape(B, T, -1, self.hd)
        cos, sin = self._tables(x, T)
        if self.hp:
            q = apply_rope(q.float(), cos, sin).to(x.dtype)
            k = apply_rope(k.float(), cos, sin).to(x.dtype)
        else:
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        q, k, v = (t.transpose(1, 2) for t in (q, k, v))
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=q.shape[1] != k.shape[1])
        return self.wo(o.transpose(1, 2).reshape(B, T, -1))

    # -- sm_100a path: residual stream x [B,T,d] bf16 -> x + attention(norm(x))
    def forward_native(self, x, norm):
        from ..ops import functional as Fn
        B, T, _ = x.shape
        hd = self.hd
        n_q, n_kv = self.wq.weight.shape[0] // hd, self.wk.weight.shape[0] // hd
        if _is_quantised(self.wq):
            # int8 / fp8 training: q|k|v are ONE quantised product (8-bit tcgen05 GEMM); the normalised
            # activations are quantised once
            from ..ops.quant import qlinear_multi
            xn = Fn.rms_norm(x, norm.weight, norm.eps)
            qkv = qlinear_multi(xn, (self.wq.weight, self.wk.weight, self.wv.weight), self.wq.mode, self.wq.block)
            cos, sin = rope_tables(T, hd, self.theta, x.device, torch.float32)
            rope = (cos.reshape(T, hd // 2), sin.reshape(T, hd // 2))
            return x + self.wo(Fn.attention_qkv(qkv, n_q, n_kv, hd, True, rope=rope))
        qkv, x = Fn.norm_linear_multi(x, norm.weight, norm.eps, (self.wq.weight, self.wk.weight, self.wv.weight),
                                      passthrough=True)
        cos, sin = rope_tables(T, hd, self.theta, x.device, torch.float32)
        rope = (cos.reshape(T, hd // 2), sin.reshape(T, hd // 2))
        return Fn.attention_proj(qkv, self.wo.weight, x, n_q, n_kv, hd, True, rope=rope)


class SwiGLU(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.w1 = nn.Linear(dim, hidden, bias=False)
        self.w3 = nn.Linear(dim, hidden, bias=False)
        self.w2 = nn.Linear(hidden, dim, bias=False)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))

    def forward_native(self, x, norm):
        """``x + mlp(norm(x))``; the norm output and the activation are recomputed in the backward."""
        from ..ops import functional as Fn
        if _is_quantised(self.w1):
            from ..ops.quant import qlinear_multi
            xn = Fn.rms_norm(x, norm.weight, norm.eps)
            gu = qlinear_multi(xn, (self.w1.weight, self.w3.weight), self.w1.mode, self.w1.block)
            return x + self.w2(Fn.swiglu_split(gu))
        if self.w1.weight.shape[0] % 128 == 0:
            return Fn.mlp_block(x, norm.weight, norm.eps, self.w1.weight, self.w3.weight, self.w2.weight)
        gu, x = Fn.norm_linear_multi(x, norm.weight, norm.eps, (self.w1.weight, self.w3.weight), passthrough=True)
        return Fn.swiglu_linear(gu, self.w2.weight, x)


class Block(nn.Module):
    def __init__(self, c: GPTConfig, layer_id: int, moe_kwargs: Optional[dict] = None):
        super().__init__()
        self.attn_norm, self.ffn_norm = RMSNorm(c.dim), RMSNorm(c.dim)
        if c.mixer == "cell":
            from .cell import CellMixer
            self.attn = CellMixer(c.dim)
        else:
            self.attn = Attention(c)
        hidden = c.mlp_hidden()
        self.is_moe = c.n_experts > 0 and layer_id % c.moe_every == 0
        self.native = c.native
        if self.is_moe:
            from ..moe import MoE
            kw = dict(moe_kwargs or {})
            kw.setdefault("grouped_mm", c.expert_grouped_mm)
            kw.setdefault("capacity_factor", c.capacity_factor)
            e_hidden = (int(hidden * c.expert_hidden_mult) + 63) // 64 * 64
            self.ffn = MoE(c.dim, e_hidden, c.n_experts, c.top_k, n_shared=c.n_shared_experts,
                           aux_coef=c.aux_coef, z_coef=c.z_coef, **kw)
        else:
            self.ffn = SwiGLU(c.dim, hidden)

    def forward(self, x):
        tp_state = getattr(self, "_fm_tp", None)
        if tp_state is not None:                 # sequence-parallel block on a row shard [Ms, d] (parallel/tp.py)
            from ..parallel import tp as fused_tp
            return fused_tp.block_forward(self, x, tp_state)
        if _native_ok(x, self.native) and hasattr(self.attn, "forward_native") and \
                isinstance(getattr(self.attn, "wq", None), nn.Linear):      # weight-only int8 modules keep their own path
            return self._forward_native(x)
        x = x + self.attn(self.attn_norm(x))
        return x + self.ffn(self.ffn_norm(x))

    def _forward_native(self, x):
        from ..ops import functional as Fn
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        x = self.attn.forward_native(x, self.attn_norm)
        if isinstance(self.ffn, SwiGLU):
            return self.ffn.forward_native(x, self.ffn_norm)
        return x + self.ffn(Fn.rms_norm(x, self.ffn_norm.weight, self.ffn_norm.eps))


class GPT(nn.Module):
    def __init__(self, c: GPTConfig, moe_kwargs: Optional[dict] = None):
        super().__init__()
        self.cfg = c
        self.tok_emb = nn.Embedding(c.vocab_size, c.dim)
        self.layers = nn.ModuleDict({str(i): Block(c, i, moe_kwargs) for i in range(c.n_layers)})
        self.norm = RMSNorm(c.dim)
        self.lm_head = nn.Linear(c.dim, c.vocab_size, bias=False)
        if c.tie_embeddings:
            self.lm_head.weight = self.tok_emb.weight
        self._reset(c)
        self._cache: dict = {}

    def _reset(self, c: GPTConfig) -> None:
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
        depth_std = 0.02 / (2 * c.n_layers) ** 0.5
        for name, p in self.named_parameters():
            if name.endswith(("wo.weight", "w2.weight")):
                nn.init.normal_(p, std=depth_std)

    # ------------------------------------------------------------------ forward
    def forward(self, tokens, labels=None):
        native = self.tok_emb is not None and _native_ok(self.tok_emb.weight, self.cfg.native) and \
            (torch.is_autocast_enabled() or self.tok_emb.weight.dtype == torch.bfloat16)
        if self.tok_emb is None:
            h = tokens
        elif native:
            from ..ops import functional as Fn
            h = Fn.embedding(tokens, self.tok_emb.weight)
        else:
            h = self.tok_emb(tokens)
        aux = None
        tp_state = getattr(self, "_fm_tp", None)
        if tp_state is not None and not isinstance(tp_state, str):
            # sequence-parallel blocks over peer memory (parallel/tp.py); weights are this rank's slices
            from ..parallel import tp as fused_tp
            h = fused_tp.stack_forward(self, h)
        else:
            for blk in self.layers.values():
                h = blk(h)
                if blk.is_moe and blk.ffn.last_aux is not None:
                    aux = blk.ffn.last_aux if aux is None else aux + blk.ffn.last_aux
        if self.lm_head is None:
            return h
        if h.is_cuda and h.dtype == torch.bfloat16 and _native_ok(h, self.cfg.native):
            from ..ops import functional as Fn
            h = Fn.rms_norm(h, self.norm.weight, self.norm.eps)
            if labels is None:
                return Fn.linear(h, self.lm_head.weight)
            ce = Fn.linear_cross_entropy(h, self.lm_head.weight, labels, self.cfg.loss_chunk)
            return ce, aux
        h = self.norm(h)
        if labels is None:
            return self.lm_head(h)
        return chunked_cross_entropy(h, self.lm_head.weight, labels, self.cfg.loss_chunk), aux

    def aux_loss(self):
        terms = [b.ffn.last_aux for b in self.layers.values() if b.is_moe and b.ffn.last_aux is not None]
        if not terms:
            return None
        total = terms[0]
        for t in terms[1:]:
            total = total + t
        return total

    # ------------------------------------------------------------------ bookkeeping
    def num_params(self, active_only: bool = False) -> int:
        key = ("n", active_only)
        if key not in self._cache:
            total = 0
            seen = set()
            for name, p in self.named_parameters():
                if id(p) in seen:
                    continue
                seen.add(id(p))
                if active_only and ".experts." in name:
                    total += p.numel() * self.cfg.top_k // self.cfg.n_experts
                else:
                    total += p.numel()
            self._cache[key] = total
        return self._cache[key]

    def flops_per_token(self, seq: int) -> int:
        """``6 * active params + 12 * layers * dim * seq`` (the reference's MFU convention,
        ``forgemind/models/gpt.py:239-246``)."""
        key = ("f", seq)
        if key not in self._cache:
            self._cache[key] = 6 * self.num_params(active_only=True) + 12 * self.cfg.n_layers * self.cfg.dim * seq
        return self._cache[key]

    def prepare(self, device=None, dtype=None, seq: Optional[int] = None) -> "GPT":
        """Build the RoPE tables (and probe the MoE dispatch path) ahead of the first step."""
        first = next(self.parameters(), None)
        device = device or (first.device if first is not None else torch.device("cpu"))
        dtype = dtype or (first.dtype if first is not None else torch.float32)
        seq = int(seq or self.cfg.max_seq)
        from ..moe import MoE
        for m in self.modules():
            if isinstance(m, Attention):
                m.cache_rope(device, dtype, seq)
                if torch.device(device).type == "cuda":
                    rope_tables(seq, m.hd, m.theta, device, torch.float32)
            elif isinstance(m, MoE):
                m.probe_grouped(device, dtype)
        return self

    def tp_plan(self) -> dict:
        return {"attn.wq": "col", "attn.wk": "col", "attn.wv": "col", "attn.wo": "row",
                "ffn.w1": "col", "ffn.w3": "col", "ffn.w2": "row"}

    def split_stage(self, stage: int, n_stages: int) -> "GPT":
        """Keep only the layers of one pipeline stage (names unchanged); first stage keeps the
        embedding, last stage the final norm and head."""
        n = self.cfg.n_layers
        sizes = [n // n_stages + (1 if s < n % n_stages else 0) for s in range(n_stages)]
        lo = sum(sizes[:stage])
        hi = lo + sizes[stage]
        for key in list(self.layers.keys()):
            if not lo <= int(key) < hi:
                del self.layers[key]
        if stage != 0:
            self.tok_emb = None
        if stage != n_stages - 1:
            self.norm = None
            self.lm_head = None
        self._cache.clear()
        return self
