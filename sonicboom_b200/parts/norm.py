"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, plain weight
(core/src/nn/norm.cpp:25-42; the model's use: core/src/model/emit.cpp:170-176, 440, 449, 512-515)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorRequest
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec, dtype, device):
        self.width, self.eps, self.tensor = spec.width, float(spec.eps), spec.tensor
        self.weight = None

    def tensor_requests(self):
        return [TensorRequest(self.tensor, (self.width,), "norm")]

    def bind(self, get):
        self.weight = get(self.tensor)

    def as_rms(self):
        return self.weight, self.eps

    def forward(self, x, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=out_dtype, device=x.device)
        return ops.rmsnorm(x, self.weight, self.eps, out, rows)
