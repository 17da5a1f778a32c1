"""An engine: one bound model, its cache, and the step function over them."""
from __future__ import annotations

import torch

from ..cache.kv import Cache
from .step import StepEntry, step


class Engine:
    """Owns the cache of a model and runs steps on it.

    `max_tokens` is the most tokens live sequences may hold together, each sequence's count
    rounded up to a whole cache page (64 tokens); it sizes the cache."""

    def __init__(self, model, max_tokens: int, n_slots: int | None = None):
        self.model = model
        self.use_decode_loop = True
        self.cache = Cache(model.kv_needs(), model.state_needs(), max_tokens,
                           dtype=model.dtype, device=model.device, n_slots=n_slots)

    def open(self) -> int:
        """A slot for a new sequence."""
        return self.cache.open()

    def close(self, slot: int) -> None:
        """Gives the sequence's slot and pages back."""
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    @property
    def page_size(self) -> int:
        return self.cache.page_size

    def free_pages(self) -> int:
        """Pages every group can still hand out."""
        return min((g.pool.free_count for g in self.cache.groups), default=0)

    def free_slots(self) -> int:
        return self.cache.slots.free_count

    def decode_loop(self, slots, budgets, samplings):
        """The captured decode step for these live sequences, or None when it cannot serve
        them (penalties need each sequence's token history on the host).  `budgets`: the most
        tokens each of them will still be asked for; each gets pages for its own budget.  A
        windowed cache group holds those pages for the life of the loop and gives back the
        ones its window has left behind when the loop is closed."""
        from .decode import DecodeLoop
        if not self.use_decode_loop or any(s.penalizes for s in samplings):
            return None
        return DecodeLoop(self, slots, budgets, samplings)

    def step(self, entries) -> torch.Tensor:
        """entries: StepEntry items or (slot, tokens, want) tuples."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(e[0], list(e[1]), list(e[2]))
                   for e in entries]
        return step(self.model, self.cache, entries)
