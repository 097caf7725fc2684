"""Parallelism strategies: data (replicated / sharded), tensor, pipeline, expert; activation checkpointing."""
from . import native  # noqa: F401
from .ac import apply_activation_checkpointing  # noqa: F401
from .pipeline import PipelineRunner  # noqa: F401
