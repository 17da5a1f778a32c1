"""Half-split (NEOX) rotary position encoding.

For pair i of the rotated prefix of a head: theta = position * exp(-2i/n * ln(base)), every
step in float32 (core/src/nn/rope.cpp:26-55); the whole head is rotated unless `rotary_dim`
names a shorter prefix (rope.cpp:58-82).  The table of per-pair frequencies is made once on
the host with the reference's operation order and handed to the rotation kernel, which is
also where a scaled-frequency variant would plug in its own table."""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope_neox")
class RotaryNeox(PositionEncoding):
    def __init__(self, spec, dtype, device):
        self.head_dim = spec.head_dim
        self.rotary_dim = spec.rotary_dim or spec.head_dim
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            from ..config.specs import ConfigError
            raise ConfigError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim "
                              f"{self.head_dim}")
        n = np.float32(self.rotary_dim)
        i = np.arange(self.rotary_dim // 2, dtype=np.float32)
        log_base = np.log(np.float32(spec.theta)).astype(np.float32)
        inv = np.exp((np.float32(-2.0) * i / n * log_base).astype(np.float32)).astype(np.float32)
        self.inv_freq = torch.from_numpy(inv).to(device)


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    """Leaves queries and keys as they are."""

    def __init__(self, spec, dtype, device):
        self.head_dim, self.rotary_dim = spec.head_dim, 0
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=device)
