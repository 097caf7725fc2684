"""Configuration dataclasses.

Field names and defaults follow the reference's ``forgemind/config.py:5-97`` so a script written
for it reads the same here. Fields that exist only in this library are grouped at the end of each
class and default to the reference's behaviour.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field


def _one_of(owner: str, name: str, value, allowed) -> None:
    if value not in allowed:
        raise ValueError(f"{owner}.{name} must be one of {', '.join(repr(a) for a in allowed)}; got {value!r}")


def _at_least(owner: str, name: str, value, low) -> None:
    if not isinstance(value, (int, float)) or isinstance(value, bool) or value < low:
        raise ValueError(f"{owner}.{name} must be a number >= {low}; got {value!r}")


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

    def check(self, world: int | None = None) -> None:
        """Raise ``ValueError`` for a mesh that cannot exist; with ``world`` also for one that does not fill it."""
        _one_of("parallel", "backend", self.backend, ("native", "deepspeed"))
        _one_of("parallel", "pp_schedule", self.pp_schedule, ("1f1b", "gpipe"))
        for name in ("dp_replicate", "tp", "pp", "ep", "pp_microbatches"):
            _at_least("parallel", name, getattr(self, name), 1)
        if self.dp_shard != -1:
            _at_least("parallel", "dp_shard", self.dp_shard, 1)
        _at_least("parallel", "comm_timeout_ms", self.comm_timeout_ms, 1)
        _at_least("parallel", "ep_slot_factor", self.ep_slot_factor, 0)
        _at_least("parallel", "fsdp_resident_bytes", self.fsdp_resident_bytes, 0)
        _one_of("parallel", "zero_stage", self.zero_stage, (0, 1, 2, 3))
        if world is not None:
            fixed = self.dp_replicate * self.tp * self.pp
            if world % fixed:
                raise ValueError(f"parallel: dp_replicate * tp * pp = {fixed} does not divide the {world} processes")
            shard = world // fixed if self.dp_shard == -1 else self.dp_shard
            if fixed * shard != world:
                raise ValueError(f"parallel: pp {self.pp} x dp_replicate {self.dp_replicate} x dp_shard {shard} x tp "
                                 f"{self.tp} = {fixed * shard} processes, but {world} were started")
            if (self.dp_replicate * shard) % self.ep:
                raise ValueError(f"parallel.ep = {self.ep} must divide dp_replicate * dp_shard = "
                                 f"{self.dp_replicate * shard}")


@dataclass
class QuantConfig:
    mode: str = "none"                 # "none" | "fp8" | "int8" | "int8_wo"
    backend: str = "auto"              # "auto" | "native" | "te" | "torchao"
    exclude: tuple = ("lm_head", "gate", "router", "tok_emb")
    optimizer_8bit: bool = False
    # ---- additions
    fp8_block: int = 128               # scale granularity of the block-scaled fp8 GEMM (1x128 act, 128x128 weight)

    def check(self) -> None:
        _one_of("quant", "mode", self.mode, ("none", "fp8", "int8", "int8_wo"))
        _one_of("quant", "backend", self.backend, ("auto", "native", "te", "torchao"))
        _at_least("quant", "fp8_block", self.fp8_block, 1)


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

    def check(self) -> None:
        _at_least("offload", "min_numel", self.min_numel, 0)
        _at_least("offload", "act_min_bytes", self.act_min_bytes, 0)
        _at_least("offload", "pipeline_chunks", self.pipeline_chunks, 1)
        if not 0.0 <= float(self.act_layers) <= 1.0:
            raise ValueError(f"offload.act_layers is the fraction of blocks to wrap, 0..1; got {self.act_layers!r}")
        if not 0.0 <= float(self.gpu_watermark) <= 1.0:
            raise ValueError(f"offload.gpu_watermark is a fraction of device memory, 0..1; got {self.gpu_watermark!r}")


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

    def check(self) -> None:
        _one_of("train", "ac", self.ac, ("none", "full", "selective"))
        _one_of("train", "optimizer", self.optimizer, ("adamw", "muon"))
        for name in ("max_steps", "warmup_steps", "eval_every", "eval_steps", "ckpt_every", "workers"):
            _at_least("train", name, getattr(self, name), 0)
        for name in ("grad_accum", "log_every", "prefetch_depth", "muon_ns_steps"):
            _at_least("train", name, getattr(self, name), 1)
        for name in ("lr", "weight_decay", "grad_clip", "skip_spike_factor", "min_lr_ratio", "muon_lr"):
            _at_least("train", name, getattr(self, name), 0)
        if len(self.betas) != 2 or not all(0.0 <= float(b) < 1.0 for b in self.betas):
            raise ValueError(f"train.betas must be two numbers in [0, 1); got {self.betas!r}")
        if not float(self.eps) > 0:
            raise ValueError(f"train.eps must be positive; got {self.eps!r}")


@dataclass
class ForgeConfig:
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    quant: QuantConfig = field(default_factory=QuantConfig)
    offload: OffloadConfig = field(default_factory=OffloadConfig)
    train: TrainConfig = field(default_factory=TrainConfig)

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    def check(self, world: int | None = None) -> "ForgeConfig":
        """Validate every section (``fm.Trainer`` calls this before it builds anything): a misspelt mode or a mesh
        that does not multiply out is reported here, by field name, instead of somewhere inside the run."""
        self.parallel.check(world)
        self.quant.check()
        self.offload.check()
        self.train.check()
        return self
