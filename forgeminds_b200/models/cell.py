"""GatedCell: a GRU-style recurrent mixer that can stand in for attention (``GPTConfig.mixer="cell"``).

``x_t [B, D]``, state ``h [B, H]`` -> new state; :meth:`GatedCell.scan` walks a sequence
``[B, T, D] -> [B, T, H]``. Mirrors the reference's ``forgemind/models/cell.py:9-52`` (same
parameters ``x2g``/``h2g``/``out`` and uniform(+-H^-0.5) init); the input projection of the whole
sequence is hoisted out of the time loop so that only the small recurrent product is sequential.
"""
from __future__ import annotations

import torch
import torch.nn as nn


class GatedCell(nn.Module):
    def __init__(self, input_dim: int, hidden_dim: int, bias: bool = True):
        super().__init__()
        self.input_dim, self.hidden_dim = input_dim, hidden_dim
        self.x2g = nn.Linear(input_dim, 3 * hidden_dim, bias=bias)     # update | reset | candidate
        self.h2g = nn.Linear(hidden_dim, 3 * hidden_dim, bias=False)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        bound = self.hidden_dim ** -0.5
        for p in self.parameters():
            nn.init.uniform_(p, -bound, bound)

    def _step(self, gx, h):
        xz, xr, xn = gx.chunk(3, dim=-1)
        hz, hr, hn = self.h2g(h).chunk(3, dim=-1)
        z = torch.sigmoid(xz + hz)
        r = torch.sigmoid(xr + hr)
        cand = torch.tanh(xn + r * hn)
        return (1 - z) * cand + z * h

    def forward(self, x, h=None):
        if h is None:
            h = x.new_zeros(x.shape[0], self.hidden_dim)
        return self._step(self.x2g(x), h)

    def scan(self, x, h=None):
        """Run the cell over ``x [B, T, D]``; returns ``(states [B, T, H], last state)``."""
        if h is None:
            h = x.new_zeros(x.shape[0], self.hidden_dim)
        gates = self.x2g(x)                       # one GEMM for all time steps
        states = []
        for t in range(x.shape[1]):
            h = self._step(gates[:, t], h)
            states.append(h)
        return torch.stack(states, dim=1), h


class CellMixer(nn.Module):
    """``[B, T, D] -> [B, T, D]`` sequence mixer built on :class:`GatedCell`."""

    def __init__(self, dim: int, hidden: int | None = None):
        super().__init__()
        self.cell = GatedCell(dim, hidden or dim)
        self.out = nn.Linear(hidden or dim, dim, bias=False)

    def forward(self, x):
        states, _ = self.cell.scan(x)
        return self.out(states)
