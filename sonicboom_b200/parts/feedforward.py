"""Dense gated feed-forward: y = Wdown (silu(Wgate f) * (Wup f)), no biases
(core/src/model/emit.cpp:364-374; silu: core/src/nn/activation.cpp:41-50).

Gate and up are one product over a fused matrix whose rows alternate in blocks of
`ops.SWIGLU_BLOCK` (8 gate rows, the 8 up rows of the same outputs, ...), so the product's
epilogue applies silu(gate) * up and writes [rows, intermediate] once; the residual add is
fused into the down projection.  These are the reference's SiluMul and ResidualAdd fusions
(core/include/sonicboom/planner/ir_passes.h:35-39)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorRequest
from .base import FeedForward, register_feed_forward


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    ff, d = gate.shape
    b = ops.SWIGLU_BLOCK
    if gate.dtype != up.dtype:
        gate, up = gate.float(), up.float()
    return torch.stack([gate.view(ff // b, b, d), up.view(ff // b, b, d)], dim=1) \
        .reshape(2 * ff, d).contiguous()


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype = spec, dtype
        if spec.activation != "silu":
            raise ConfigError(f"feed-forward activation {spec.activation!r} is not built (only silu)")
        if spec.intermediate % ops.SWIGLU_BLOCK:
            raise ConfigError(f"intermediate_size {spec.intermediate} must be a multiple of "
                              f"{ops.SWIGLU_BLOCK} for the fused gate/up product")
        self.w_gate_up = self.w_down = None

    def tensor_requests(self):
        p, d, ff = self.spec.prefix, self.spec.width, self.spec.intermediate
        return [TensorRequest(p + "gate_proj.weight", (ff, d)),
                TensorRequest(p + "up_proj.weight", (ff, d)),
                TensorRequest(p + "down_proj.weight", (d, ff))]

    def bind(self, get):
        p = self.spec.prefix
        self.w_gate_up = interleave_gate_up(get(p + "gate_proj.weight"), get(p + "up_proj.weight"))
        self.w_down = get(p + "down_proj.weight")

    def forward(self, h, ctx, residual=None):
        rows = h.shape[0]
        t = torch.empty((rows, self.spec.intermediate), dtype=self.dtype, device=h.device)
        ops.linear(h, self.w_gate_up, t, ops.EPI_SWIGLU)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(t, self.w_down, out,
                          ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)
