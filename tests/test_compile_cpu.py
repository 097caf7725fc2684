"""`train.compile` on CPU: the blocks compile as whole graphs and train like the eager model.

The counterpart of the reference's compile conformance tests (`tests/test_compile.py`), with
`aot_eager` standing in for inductor. On a B200 the hot path does not use `torch.compile`; the
option belongs to the library engine and is kept for parity.
"""
import pytest
import torch

import forgeminds_b200 as fm


def _run(compile_on: bool, moe: bool = False):
    torch.manual_seed(0)
    cfg = fm.ForgeConfig()
    cfg.train.__dict__.update(max_steps=4, grad_accum=1, lr=3e-3, warmup_steps=1, bf16=False, resume=False,
                              log_every=1000, prefetch=False, compile=compile_on, compile_backend="aot_eager",
                              compile_fullgraph=not moe)
    extra = dict(n_experts=4, top_k=2) if moe else {}
    mc = fm.GPTConfig(vocab_size=64, dim=32, n_layers=2, n_heads=2, n_kv_heads=1, max_seq=16, ffn_hidden=64, **extra)
    tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(64, 16, n=256), micro_batch=8)
    try:
        return [h["loss"] for h in tr.fit()]
    finally:
        tr.close()


def test_dense_blocks_compile_fullgraph_and_match_eager():
    eager, compiled = _run(False), _run(True)
    assert compiled[-1] < compiled[0]
    assert eager == pytest.approx(compiled, rel=1e-4, abs=1e-4)


def test_moe_blocks_compile_with_graph_breaks_allowed():
    eager, compiled = _run(False, moe=True), _run(True, moe=True)
    assert eager == pytest.approx(compiled, rel=1e-3, abs=1e-3)
