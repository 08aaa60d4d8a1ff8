"""Rotary position encoding (crates/cellm-kernels/src/cpu_kernels.rs:264-292):
pairs (i, i + rot/2) ("half") or (2i, 2i+1) ("interleaved") of the first
`rotary_dim` values of a head turn by pos * theta^(-2i/rotary_dim)."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from .base import Position
from .registry import register_position


class RotaryEmbedding(Position):
    graph_safe = True

    """params: head_dim, rotary_dim, theta, layout ("half" | "interleaved")."""

    def __init__(self, params: dict, device):
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.layout = params.get("layout", "half")
        if self.layout not in ("half", "interleaved"):
            raise ConfigError(f"rope: layout {self.layout!r} is neither 'half' nor 'interleaved'")
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ConfigError(f"rope: rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = (self.theta ** (-(2.0 * i) / self.rotary_dim)).to(device)

    def rotation(self):
        return self.rotary_dim, self.layout == "interleaved", self.inv_freq


register_position("rope", RotaryEmbedding)
