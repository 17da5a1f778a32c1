"""Grouped-query attention over the paged cache, the mixer of this architecture.

Order of operations as the reference's emitter writes it (core/src/model/emit.cpp:255-308):
q = Wq h + bq; rotate q; k = Wk h, v = Wv h, then their biases; rotate k; store k, v; attend
with scale applied after the dot and a causal (optionally windowed) mask
(core/src/nn/attention.cpp:26-105); output projection (without bias in this architecture; a
spec may ask for one); the residual add is fused into that projection.  The three input projections are one product over a fused
[q | k | v] matrix, the way the reference reads "sibling" weights in one launch
(core/src/quant/mmvq_q8_1.cuh:634).  An entry that reads another entry's cache projects
queries only."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.kv import KVNeed
from ..weights.loader import TensorRequest
from .base import POSITION_ENCODINGS, Mixer, make, register_mixer


@register_mixer("attention")
class Attention(Mixer):
    def __init__(self, spec, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.hq, self.hkv, self.hd = spec.n_heads, spec.n_kv_heads, spec.head_dim
        self.qw, self.kvw = self.hq * self.hd, self.hkv * self.hd
        if self.hq % self.hkv:
            from ..config.specs import ConfigError
            raise ConfigError(f"{self.hq} query heads are not a multiple of {self.hkv} key/value heads")
        self.position = make(POSITION_ENCODINGS, "position encoding", spec.position, dtype, device)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def kv_need(self):
        return KVNeed(self.hkv, self.hd, self.spec.window)

    def tensor_requests(self):
        p, d = self.spec.prefix, self.spec.width
        req = [TensorRequest(p + "q_proj.weight", (self.qw, d)),
               TensorRequest(p + "k_proj.weight", (self.kvw, d)),
               TensorRequest(p + "v_proj.weight", (self.kvw, d)),
               TensorRequest(p + "o_proj.weight", (d, self.qw))]
        if self.spec.qkv_bias:
            req += [TensorRequest(p + "q_proj.bias", (self.qw,), "bias"),
                    TensorRequest(p + "k_proj.bias", (self.kvw,), "bias"),
                    TensorRequest(p + "v_proj.bias", (self.kvw,), "bias")]
        if self.spec.out_bias:
            req.append(TensorRequest(p + "o_proj.bias", (d,), "bias"))
        return req

    def bind(self, get):
        p = self.spec.prefix
        self.w_qkv = _cat([get(p + f"{n}_proj.weight") for n in "qkv"])
        if self.spec.qkv_bias:
            self.b_qkv = _cat([get(p + f"{n}_proj.bias") for n in "qkv"])
        self.w_o = get(p + "o_proj.weight")
        if self.spec.out_bias:
            self.b_o = get(p + "o_proj.bias")

    def first_weights(self, rows):
        n, k = self.w_qkv.shape
        late = self.w_qkv.dtype == torch.bfloat16 and ops.requests_weights_late(rows, n, k, self.w_qkv.device)
        return self.w_qkv if late else None

    def forward(self, h, ctx, residual=None):
        rows = h.shape[0]
        plan = ctx.plan
        width_in = self.qw + (2 * self.kvw if ctx.owns_cache else 0)
        storage = ctx.kv_storage()
        g = plan.groups[ctx.kv_group()]
        q = torch.empty((rows, self.hq, self.hd), dtype=self.dtype, device=h.device)
        ops.qkv_rope_store(h, self.w_qkv[:width_in],
                           self.b_qkv[:width_in] if self.b_qkv is not None else None, self.hq, self.hkv,
                           self.hd, self.position.rotary_dim, self.position.inv_freq, plan.row_seq,
                           plan.row_pos, g.page_off, g.page_ids, g.page_size,
                           storage if ctx.owns_cache else None, q)
        mixed = torch.empty((rows, self.qw), dtype=self.dtype, device=h.device)
        ops.attention(q, mixed, plan, ctx.kv_group(), storage, self.hq, self.hkv, self.hd,
                      self.spec.window, self.spec.scale, warm=self.w_o)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        epilogue = ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE
        if self.b_o is None:
            return ctx.linear(mixed, self.w_o, out, epilogue, residual=residual, act_dtype=self.dtype)
        # with an output bias (not this architecture's): the bias follows the product as a step
        # of its own, so no norm rides on the product
        ops.linear(mixed, self.w_o, out, epilogue, residual=residual)
        return ops.add_bias(out, self.b_o)


def _cat(tensors):
    """Rows of several tensors in one; a mix of kept dtypes goes to the widest."""
    if len({t.dtype for t in tensors}) > 1:
        tensors = [t.float() for t in tensors]
    return torch.cat(tensors, dim=0).contiguous()
