"""Fused tensor parallelism (all-gather -> GEMM, GEMM -> reduce-scatter over peer memory)."""
from __future__ import annotations


def usable(ctx) -> bool:
    return False
