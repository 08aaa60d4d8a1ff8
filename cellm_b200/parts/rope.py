"""Rotary position encoding (crates/cellm-kernels/src/cpu_kernels.rs:264-292):
pairs (i, i + rot/2) ("half") or (2i, 2i+1) ("interleaved") of the first
`rotary_dim` values of a head turn by pos * theta^(-2i/rotary_dim)."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from .base import Position
from .registry import register_position


def split_inv_freq(theta: float, rotary_dim: int) -> torch.Tensor:
    """theta^(-2i/rotary_dim) for i < rotary_dim/2, computed in 64-bit and given as
    [rotary_dim/2, 2] float32: the nearest float and the remainder, so that the
    kernel can form pos * inv_freq without losing the low bits."""
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    inv = float(theta) ** (-(2.0 * i) / max(rotary_dim, 1))
    hi = inv.to(torch.float32)
    lo = (inv - hi.to(torch.float64)).to(torch.float32)
    return torch.stack([hi, lo], dim=1).contiguous()


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
        self.inv_freq = split_inv_freq(self.theta, self.rotary_dim).to(device)

    def rotation(self):
        return self.rotary_dim, self.layout == "interleaved", self.inv_freq


register_position("rope", RotaryEmbedding)
