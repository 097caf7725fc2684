"""forgeminds_b200: a Blackwell-first training library.

Three entry levels, as in the reference (``forgemind/__init__.py:1-41``):

* :class:`Trainer` -- config-driven full stack (``ForgeConfig`` mesh of
  ``pp x dp_replicate x dp_shard x tp`` with ``ep``; quantisation, offload, checkpoints);
* :class:`Forge` -- a two-line facade for any ``nn.Module``;
* plain functions -- :func:`launch`, :func:`all_reduce` / :func:`broadcast` / :func:`all_gather` /
  :func:`barrier`, :func:`seed_everything`.

``import forgeminds_b200`` stays light: the kernel package, the autotuner, the composable blocks
and Muon are loaded on first attribute access, and neither the native extension nor
``torch._dynamo`` is imported until something needs it.
"""
from __future__ import annotations

import importlib

from .config import ForgeConfig, OffloadConfig, ParallelConfig, QuantConfig, TrainConfig
from .data import BatchStream, RandomTokens, ResumableSampler, SyntheticLM, TokenFile, async_loader, build_loader, to_device
from .distributed import DistContext, all_gather, all_reduce, barrier, broadcast, cleanup, init_distributed
from .forge import Forge, launch, seed_everything
from .models.gpt import GPT, GPTConfig
from .moe import MoE
from .offload import OffloadedAdamW
from .perf import count_host_syncs, host_syncs
from .trainer import Trainer, moe_kwargs

__version__ = "0.1.0"

_LAZY_MODULES = ("kernels", "autotune", "nn", "muon", "ops", "quant", "parallel")


def __getattr__(name: str):
    if name in _LAZY_MODULES:
        mod = importlib.import_module(f"{__name__}.{name}")
        globals()[name] = mod
        return mod
    if name == "Muon":
        from .muon import Muon
        globals()["Muon"] = Muon
        return Muon
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = [
    "ForgeConfig", "ParallelConfig", "QuantConfig", "OffloadConfig", "TrainConfig",
    "init_distributed", "DistContext", "cleanup", "Trainer", "moe_kwargs", "GPT", "GPTConfig", "MoE",
    "OffloadedAdamW", "SyntheticLM", "TokenFile", "RandomTokens", "BatchStream", "ResumableSampler",
    "build_loader", "async_loader", "to_device", "count_host_syncs", "host_syncs", "Forge", "launch",
    "seed_everything", "Muon", "all_reduce", "all_gather", "broadcast", "barrier",
]
