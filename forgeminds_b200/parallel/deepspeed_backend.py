"""DeepSpeed back end: JSON config builder and engine bring-up (``ParallelConfig.backend="deepspeed"``).

Only :func:`build_ds_config` runs without the ``deepspeed`` package; the other helpers import it
lazily and raise a clear error when it is missing. Keys and rules follow the reference's
``forgemind/parallel/deepspeed_backend.py:9-66`` (ZeRO 1/2/3, optimizer/parameter CPU offload,
AutoTP, bf16, gradient clipping; pipeline parallelism requires ZeRO stage <= 1).
"""
from __future__ import annotations

from ..config import ForgeConfig


def build_ds_config(cfg: ForgeConfig, world: int, micro_batch: int) -> dict:
    pc, tc = cfg.parallel, cfg.train
    if pc.pp > 1 and pc.zero_stage > 1:
        raise ValueError("DeepSpeed pipeline parallelism supports ZeRO stage 0/1 only")
    dp = max(1, world // (pc.tp * pc.pp))
    zero = {"stage": int(pc.zero_stage), "overlap_comm": True, "contiguous_gradients": True,
            "reduce_bucket_size": int(5e8), "allgather_bucket_size": int(5e8)}
    if pc.zero_offload_optimizer:
        zero["offload_optimizer"] = {"device": "cpu", "pin_memory": True}
    if pc.zero_offload_param:
        if pc.zero_stage != 3:
            raise ValueError("parameter offload needs ZeRO stage 3")
        zero["offload_param"] = {"device": "cpu", "pin_memory": True}
    if pc.zero_stage == 3:
        zero["stage3_gather_16bit_weights_on_model_save"] = True
    out = {
        "train_micro_batch_size_per_gpu": int(micro_batch),
        "gradient_accumulation_steps": int(tc.grad_accum),
        "train_batch_size": int(micro_batch) * int(tc.grad_accum) * dp,
        "gradient_clipping": float(tc.grad_clip),
        "bf16": {"enabled": bool(tc.bf16)},
        "zero_optimization": zero,
        "steps_per_print": int(1e9),
        "wall_clock_breakdown": False,
    }
    if pc.tp > 1:
        out["tensor_parallel"] = {"autotp_size": int(pc.tp)}
    out.update(pc.ds_extra or {})
    return out


def _deepspeed():
    try:
        import deepspeed
    except ImportError as exc:
        raise RuntimeError("ParallelConfig.backend='deepspeed' needs the deepspeed package") from exc
    return deepspeed


def to_pipeline_module(model, n_stages: int):
    """Flatten a GPT into a ``deepspeed.pipe.PipelineModule`` (embedding, blocks, norm, head)."""
    ds = _deepspeed()
    from deepspeed.pipe import PipelineModule
    layers = [model.tok_emb, *model.layers.values(), model.norm, model.lm_head]
    return PipelineModule(layers=layers, num_stages=n_stages, partition_method="parameters")


def init_deepspeed(model, param_groups, cfg: ForgeConfig, world: int, micro_batch: int):
    ds = _deepspeed()
    ds_cfg = build_ds_config(cfg, world, micro_batch)
    tc = cfg.train
    if cfg.parallel.zero_offload_optimizer:
        from deepspeed.ops.adam import DeepSpeedCPUAdam as Adam
        opt = Adam(param_groups, lr=tc.lr, betas=tc.betas, eps=tc.eps)
    else:
        from deepspeed.ops.adam import FusedAdam as Adam
        opt = Adam(param_groups, lr=tc.lr, betas=tc.betas, eps=tc.eps, adam_w_mode=True)
    if cfg.parallel.pp > 1:
        model = to_pipeline_module(model, cfg.parallel.pp)
    engine, opt, _, _ = ds.initialize(model=model, optimizer=opt, config=ds_cfg)
    return engine, opt
