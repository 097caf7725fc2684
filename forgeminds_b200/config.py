"""Configuration dataclasses.

Field names and defaults follow the reference's ``forgemind/config.py:5-97`` so a script written
for it reads the same here. Fields that exist only in this library are grouped at the end of each
class and default to the reference's behaviour.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field


@dataclass
class ParallelConfig:
    """Device mesh: ``world = pp * dp_replicate * dp_shard * tp``; ``dp_shard=-1`` takes the rest.

    ``ep`` groups are cut out of consecutive data-parallel ranks and must divide
    ``dp_replicate * dp_shard``.
    """
    backend: str = "native"            # "native" | "deepspeed" (config builder only, library optional)
    dp_replicate: int = 1
    dp_shard: int = 1
    tp: int = 1
    pp: int = 1
    ep: int = 1
    pp_microbatches: int = 4
    pp_schedule: str = "1f1b"          # "1f1b" | "gpipe"
    fsdp_reshard_after_forward: bool = True
    fsdp_cpu_offload: bool = False
    ddp_static_graph: bool = False
    init_timeout_s: int = 1800
    zero_stage: int = 2
    zero_offload_optimizer: bool = False
    zero_offload_param: bool = False
    ds_extra: dict = field(default_factory=dict)
    # ---- additions of this library
    fused_comm: bool = True            # use the peer-memory kernels (falls back to torch.distributed when unavailable)
    fsdp_resident_bytes: int = 0       # memory the flat-store engine may use for parameters, gradients and optimizer
                                       # state on one GPU (0: 80 % of the device); bigger models go to FSDP2
    comm_timeout_ms: int = 10000       # bound of every device-side wait on a peer flag
    ep_slot_factor: float = 0.0        # dropless expert parallelism: row buffers of a rank hold this many times its
                                       # average share of the routed rows (0: the worst case, every row); a layer
                                       # that needs more raises fm.ops.EPOverflow at the step's host read


@dataclass
class QuantConfig:
    mode: str = "none"                 # "none" | "fp8" | "int8" | "int8_wo"
    backend: str = "auto"              # "auto" | "native" | "te" | "torchao"
    exclude: tuple = ("lm_head", "gate", "router", "tok_emb")
    optimizer_8bit: bool = False
    # ---- additions
    fp8_block: int = 128               # scale granularity of the block-scaled fp8 GEMM (1x128 act, 128x128 weight)


@dataclass
class OffloadConfig:
    optimizer: bool = False
    smart: bool = True
    min_numel: int = 1 << 18
    gpu_watermark: float = 0.0
    activations: bool = False
    act_min_bytes: int = 1 << 20
    act_layers: float = 1.0
    act_pool: bool = True
    pipeline_chunks: int = 4
    experts: bool = False


@dataclass
class TrainConfig:
    max_steps: int = 1000
    grad_accum: int = 1
    lr: float = 3e-4
    min_lr_ratio: float = 0.1
    warmup_steps: int = 100
    weight_decay: float = 0.1
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-8
    grad_clip: float = 1.0
    bf16: bool = True
    compile: bool = False
    compile_mode: str = "default"
    compile_backend: str = "inductor"
    compile_fullgraph: bool = False
    ac: str = "none"                   # "none" | "full" | "selective"
    ac_preserve_rng: bool = False
    seed: int = 1234
    log_every: int = 10
    eval_every: int = 0
    eval_steps: int = 20
    ckpt_every: int = 0
    ckpt_dir: str = "checkpoints"
    resume: bool = True
    skip_spike_factor: float = 0.0
    skip_nonfinite: bool = True
    prefetch: bool = True
    prefetch_depth: int = 2
    batch_thread: bool | None = None
    workers: int = 0
    fused_ops: bool = False
    fused_split_mlp: bool = False
    # ---- additions
    optimizer: str = "adamw"           # "adamw" | "muon" (Muon on 2-D block weights, AdamW elsewhere)
    native: bool | None = None         # None = use the sm_100a engine when the device is a CUDA GPU and bf16 is on
    muon_lr: float = 0.02
    muon_momentum: float = 0.95
    muon_ns_steps: int = 5


@dataclass
class ForgeConfig:
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    quant: QuantConfig = field(default_factory=QuantConfig)
    offload: OffloadConfig = field(default_factory=OffloadConfig)
    train: TrainConfig = field(default_factory=TrainConfig)

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)
