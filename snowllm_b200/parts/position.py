"""Position encodings of the rotary family: a table of inverse frequencies and how many of a
head's elements rotate.  inv_freq[i] = theta^(-2i/rot_dim) in float
(snowllm/models/lfm2/layers.py:116-117); the angle pos * inv_freq[i] is formed in float inside the
kernel that applies it."""
from __future__ import annotations

import torch

from .registry import register_position


class RotaryPosition:
    def __init__(self, *, head_dim: int, theta: float, rot_dim: int | None = None):
        self.head_dim, self.theta = head_dim, float(theta)
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ValueError(f"rot_dim={self.rot_dim} must be even and at most head_dim={head_dim}")
        self._inv_freq = None

    def rotary(self, device):
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            inv = 1.0 / (self.theta ** (torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / self.rot_dim))
            self._inv_freq = inv.to(device)
        return self._inv_freq, self.rot_dim


class NoPosition:
    """No position encoding (the mixer sees order only through its causal mask)."""

    def __init__(self, **_):
        pass

    def rotary(self, device):
        return None, 0


register_position("rope", RotaryPosition)
register_position("none", NoPosition)
