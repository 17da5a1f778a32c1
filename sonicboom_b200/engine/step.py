"""The step function: a batch of sequences, their next tokens in one pass over the model.

The reference runs one sequence at a time through two graphs: a prefill graph over
`tokens[n]` from `start_pos` (core/src/model/emit.cpp:649-652, 824-837) and a decode graph
over one token at `pos` (emit.cpp:500-501, 800-822).  Here one function does both for a
batch: every entry brings a slot and that sequence's next tokens (a whole prompt, or one
token, or any other cut), the rows of all entries are packed into one batch, keys and values
are written into each sequence's pages at its own positions, and logits come back for the
rows that were asked for.  It runs only the tokens it is given; everything earlier is read
from the cache.  Rows are packed without padding, so padding cannot change a result.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .. import ops
from ..cache.kv import Cache


class StepError(ValueError):
    pass


@dataclass
class StepEntry:
    slot: int
    tokens: list            # next token ids of the sequence in this slot
    want: list = field(default_factory=list)   # places among `tokens` whose logits are wanted


@dataclass
class GroupPlan:
    page_off: torch.Tensor  # int32 [n_seqs + 1]
    page_ids: torch.Tensor  # int32 [pages of all sequences], -1 where a page was given back
    page_size: int


class StepPlan:
    """Device-side description of one step: int32 arrays every kernel indexes by row or by
    sequence.  Built on the host, copied with one transfer."""

    def __init__(self, cache: Cache, entries: list[StepEntry], device):
        n_seqs = len(entries)
        lens = [len(e.tokens) for e in entries]
        pos0 = [cache.length(e.slot) for e in entries]
        n_rows = sum(lens)
        self.n_rows, self.n_seqs = n_rows, n_seqs
        self.max_new = max(lens)
        self.max_len = max(p + n for p, n in zip(pos0, lens))
        row0 = np.zeros(n_seqs + 1, dtype=np.int32)
        row0[1:] = np.cumsum(lens)
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        row_seq = np.repeat(np.arange(n_seqs, dtype=np.int32), lens)
        row_pos = np.concatenate([np.arange(p, p + n, dtype=np.int32) for p, n in zip(pos0, lens)])
        want = np.asarray([row0[i] + w for i, e in enumerate(entries) for w in e.want],
                          dtype=np.int32)
        self.n_want = int(want.size)
        parts = [tokens, row_seq, row_pos, row0, np.asarray(pos0, dtype=np.int32),
                 np.asarray([e.slot for e in entries], dtype=np.int32), want]
        for gi in range(len(cache.groups)):
            lists = [cache.page_list(e.slot, gi) for e in entries]
            off = np.zeros(n_seqs + 1, dtype=np.int32)
            off[1:] = np.cumsum([len(l) for l in lists])
            ids = np.asarray([p for l in lists for p in l], dtype=np.int32)
            parts += [off, ids]
        # every section starts on a 16-byte boundary so that kernels may use vector loads
        padded = [np.concatenate([p, np.zeros(-p.size % 4, dtype=np.int32)]) for p in parts]
        flat = np.concatenate(padded)
        host = torch.from_numpy(flat)
        if torch.device(device).type == "cuda":
            host = host.pin_memory()
        dev = host.to(device, non_blocking=True)
        self._host = host
        views, at = [], 0
        for p, q in zip(parts, padded):
            views.append(dev[at:at + p.size])
            at += q.size
        (self.tokens, self.row_seq, self.row_pos, self.seq_row0, self.seq_pos0, self.seq_slot,
         self.want_rows) = views[:7]
        self.groups = [GroupPlan(views[7 + 2 * gi], views[8 + 2 * gi], cache.page_size)
                       for gi in range(len(cache.groups))]
        self.host_row_pos = row_pos
        self._scratch = None

    def scratch(self, nbytes: int, device):
        """Scratch memory shared by the step's kernels (made on first use, grown on demand);
        None when nothing is asked for."""
        if nbytes <= 0:
            return None
        if self._scratch is None or self._scratch.numel() < nbytes:
            self._scratch = torch.empty(nbytes, dtype=torch.uint8, device=device)
        return self._scratch


def validate(cache: Cache, entries: list[StepEntry], vocab: int, max_positions: int) -> None:
    """Host-side refusals, before anything is launched or reserved."""
    if not entries:
        raise StepError("a step needs at least one entry")
    seen = set()
    for e in entries:
        if e.slot in seen:
            raise StepError(f"slot {e.slot} appears twice in one step")
        seen.add(e.slot)
        if e.slot not in cache.records:
            raise StepError(f"slot {e.slot} holds no sequence")
        n = len(e.tokens)
        if n == 0:
            raise StepError(f"slot {e.slot}: an entry needs at least one token")
        bad = [t for t in e.tokens if not 0 <= int(t) < vocab]
        if bad:
            raise StepError(f"slot {e.slot}: token id {bad[0]} is outside the vocabulary of {vocab}")
        if cache.length(e.slot) + n > max_positions:
            raise StepError(f"slot {e.slot}: {cache.length(e.slot)} + {n} tokens exceed "
                            f"max_position_embeddings = {max_positions}")
        for w in e.want:
            if not 0 <= w < n:
                raise StepError(f"slot {e.slot}: wanted place {w} is outside its {n} tokens")


def step(model, cache: Cache, entries: list[StepEntry]) -> torch.Tensor:
    """Runs one step; returns float32 logits [wanted rows, vocab] on the device, in the order
    of the entries and of their `want` lists (None when nothing is wanted)."""
    validate(cache, entries, model.spec.vocab, model.spec.max_positions)
    for e in entries:
        cache.reserve(e.slot, cache.length(e.slot) + len(e.tokens))
    plan = StepPlan(cache, entries, model.device)
    with ops.trace_range(f"step ({plan.n_rows} rows, {plan.n_seqs} sequences)"):
        logits = model.forward(plan, cache)
    for e in entries:
        cache.advance(e.slot, cache.length(e.slot) + len(e.tokens))
    return logits
