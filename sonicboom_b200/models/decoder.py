"""The decoder as a whole: embedding, the blocks in schedule order, final norm, LM head.

One class serves every architecture that can be written as a `ModelSpec`; what differs
between architectures is the spec, not this code.  Order as the reference's emitter walks a
recipe (core/src/model/emit.cpp:237-247 embedding with its optional scale, 436-459 blocks,
512-523 head with its optional logit cap; both are fields of the spec, as the reference keeps
them as traits, core/src/model/recipe.cpp:35-61): the head
runs only on the rows whose logits are wanted (the reference takes the last row only,
core/src/model/gemma4_plan.cpp:599-605), and a tied head reads the embedding matrix
(core/src/model/exec.cpp:516-517).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import ModelSpec
from ..parts import BLOCKS, NORMS, StepContext, make
from ..weights.loader import TensorRequest


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, not {dtype}")
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.blocks = [make(BLOCKS, "block arrangement", l, dtype, device)
                       for l in spec.layers]
        self.final_norm = make(NORMS, "norm", spec.final_norm, dtype, device)
        for i, e in enumerate(spec.schedule):
            if e.cache_from is not None:
                mine = self.blocks[e.layer].kv_need()
                theirs = self.blocks[spec.schedule[e.cache_from].layer].kv_need()
                if mine != theirs:
                    from ..config.specs import ConfigError
                    raise ConfigError(f"schedule[{i}] reads the cache of entry {e.cache_from}, "
                                      f"whose keys and values ({theirs}) are not what it needs ({mine})")
        self.embedding = self.head = None

    # ------------------------------------------------------------------ weights
    def tensor_requests(self) -> list[TensorRequest]:
        s = self.spec
        req = [TensorRequest(s.embedding_tensor, (s.vocab, s.width), "embedding")]
        for b in self.blocks:
            req += b.tensor_requests()
        req += self.final_norm.tensor_requests()
        if s.head_tensor is not None:
            req.append(TensorRequest(s.head_tensor, (s.vocab, s.width)))
        else:
            # a tied model's file may still carry a copy of the head; it is not read
            req.append(TensorRequest("lm_head.weight", (s.vocab, s.width), optional=True))
        return req

    def bind(self, get) -> None:
        self.embedding = get(self.spec.embedding_tensor)
        for b in self.blocks:
            b.bind(get)
        self.final_norm.bind(get)
        self.head = self.embedding if self.spec.head_tensor is None else get(self.spec.head_tensor)

    # ------------------------------------------------------------------ what the cache must hold
    def kv_needs(self) -> list:
        """Per schedule entry: its KVNeed, or None when it reads another entry's cache."""
        return [self.blocks[e.layer].kv_need() if e.cache_from is None else None
                for e in self.spec.schedule]

    def state_needs(self) -> list:
        return [self.blocks[e.layer].state_need() for e in self.spec.schedule]

    # ------------------------------------------------------------------ one step
    def forward(self, plan, cache) -> torch.Tensor:
        """Runs the step's rows through every schedule entry; returns float32 logits
        [len(plan.want_rows), vocab] (None when no logits are wanted)."""
        s = self.spec
        x = torch.empty((plan.n_rows, s.width), dtype=torch.float32, device=self.device)
        ops.embed(plan.tokens, self.embedding, x, s.embedding_scale)
        ctx = StepContext(plan=plan, cache=cache)
        for i, e in enumerate(s.schedule):
            ctx.entry = i
            ctx.owns_cache = e.cache_from is None
            ctx.kv_entry = i if e.cache_from is None else e.cache_from
            # the next entry's first norm can ride on this entry's last product
            nxt = self.blocks[s.schedule[i + 1].layer] if i + 1 < len(s.schedule) else None
            ctx.after_block_norm = nxt.input_norm() if nxt is not None else None
            # ... and its first weights can be asked into L2 meanwhile, if it would ask late
            ctx.after_block_weights = nxt.first_weights(plan.n_rows) if nxt is not None else None
            with ops.trace_range(f"entry {i} (layer {e.layer})"):
                x = self.blocks[e.layer].forward(x, ctx)
        if plan.n_want == 0:
            return None
        hn = self.final_norm.forward(x, self.dtype, rows=plan.want_rows)
        logits = torch.empty((plan.n_want, s.vocab), dtype=torch.float32, device=self.device)
        ops.linear(hn, self.head, logits)
        return ops.softcap(logits, s.logit_cap) if s.logit_cap > 0.0 else logits


def tensor_requests(spec: ModelSpec) -> list[TensorRequest]:
    """Tensors a model of this spec wants; no device is touched."""
    return DecoderModel(spec, torch.float32, "cpu").tensor_requests()
