"""The decode loop on the device: one captured CUDA graph per batch, replayed once a token.

The reference captures its decode step as a CUDA graph and replays it per token, feeding each
argmax back through device memory (`greedy_step`: set the position, one cudaGraphLaunch, read
the token; core/src/model/gemma4_plan.cpp:1650-1696, core/include/sonicboom/hal/command.h:
34-45).  The same is done here for a batch: the step's plan lives in persistent device
buffers; the graph runs the model's own step (the same parts and kernels as an eager step),
the sampler, which writes the new tokens where the next step's embedding reads them, and a
one-line kernel that advances the positions.  Pages for all tokens the loop may produce are
reserved up front, each row for its own budget, so the page tables in the graph stay valid.

A row that has finished stays in the captured batch until the batch is captured again.  It
cannot leave its own pages: the kernel that advances the positions stops every row at the last
position it has reserved (`row_last`), and the kernels that write and read the cache check a
position against the sequence's own page list.  The reference never steps a finished sequence
again (core/include/sonicboom/model/plan.h:438-440) and refuses what does not fit its context
instead of wrapping (core/src/model/gemma4_plan.cpp:7334); both hold here per row.

`run_device` replays with no host work in between; `step_host` is the serving form: the
step's token ids are copied from pinned host memory, the graph is replayed, and the new ids
are read back.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..sampling.params import Sampling
from ..sampling.sampler import pack_params
from .step import GroupPlan


class DecodePlan:
    """A step plan of one token per sequence in buffers that outlive the step."""

    def __init__(self, cache, slots, last_positions, device):
        n = len(slots)
        lengths = [cache.length(s) for s in slots]
        self.n_rows = self.n_seqs = self.n_want = n
        self.max_new = 1
        ar = torch.arange(n + 1, dtype=torch.int32)
        self.tokens = torch.zeros(n, dtype=torch.int32, device=device)
        self.row_seq = ar[:n].to(device)
        self.row_pos = torch.tensor(lengths, dtype=torch.int32, device=device)
        self.row_last = torch.tensor(list(last_positions), dtype=torch.int32, device=device)
        self.seq_row0 = ar.to(device)
        self.seq_pos0 = self.row_pos                       # one new row per sequence
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=device)
        self.want_rows = self.row_seq
        self.groups = []
        self.max_len = 0
        for gi in range(len(cache.groups)):
            lists = [cache.page_list(s, gi) for s in slots]
            off = np.zeros(n + 1, dtype=np.int32)
            off[1:] = np.cumsum([len(l) for l in lists])
            ids = np.asarray([p for l in lists for p in l], dtype=np.int32)
            self.groups.append(GroupPlan(torch.from_numpy(off).to(device),
                                         torch.from_numpy(ids).to(device), cache.page_size))
            self.max_len = max(self.max_len, max(len(l) for l in lists) * cache.page_size)
        self._scratch = None

    def scratch(self, nbytes: int, device):
        if nbytes <= 0:
            return None
        if self._scratch is None or self._scratch.numel() < nbytes:
            self._scratch = torch.empty(nbytes, dtype=torch.uint8, device=device)
        return self._scratch


STATUS_EVERY = 64      # steps between looks at the kernels' status words in `step_host`


class DecodeLoop:
    def __init__(self, engine, slots, budgets, samplings=None, use_graph: bool = True):
        """`slots`: live sequences that have been prefilled; `budgets`: how many tokens the loop
        may be asked to produce for each of them (one number for all, or one per slot).  Every
        slot gets pages for its own budget and no more; nothing is reserved when the cache
        cannot supply all of them (CacheFull)."""
        cache, model = engine.cache, engine.model
        self.engine, self.slots, self.device = engine, list(slots), model.device
        n = len(self.slots)
        if isinstance(budgets, int):
            budgets = [budgets] * n
        self.budgets = [int(b) for b in budgets]
        if len(self.budgets) != n or min(self.budgets, default=0) < 1:
            raise ValueError(f"{n} slots need {n} budgets of at least one token, got {budgets}")
        self.start = [cache.length(s) for s in self.slots]
        for s, at, b in zip(self.slots, self.start, self.budgets):
            if at + b > model.spec.max_positions:
                raise ValueError(f"slot {s}: {at} + {b} tokens exceed max_position_embeddings = "
                                 f"{model.spec.max_positions}")
        cache.reserve_many([(s, at + b) for s, at, b in zip(self.slots, self.start, self.budgets)])
        self.max_new, self.done = max(self.budgets), 0
        self.fed = [0] * n              # steps each row took part in while it was live
        self.live = [True] * n
        self.plan = DecodePlan(cache, self.slots,
                               [at + b - 1 for at, b in zip(self.start, self.budgets)], self.device)
        samplings = samplings or [Sampling().checked()] * n
        if any(s.penalizes for s in samplings):
            raise ValueError("the device decode loop keeps no token history for penalties")
        rec, _ = pack_params(samplings, [0] * n, [[]] * n)
        self.params = torch.from_numpy(rec).to(self.device)
        self.host_in = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.host_out = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.h2d_bytes_per_step = self.d2h_bytes_per_step = 4 * n
        self.graph = None
        before = ops.LAUNCHES
        # One eager run first: it builds what is built lazily and sets kernel attributes, which
        # cannot happen inside a capture.  It must leave the sequences as it found them: the
        # keys and values it writes at the current positions are overwritten by the first real
        # step, and the slots' rows of every fixed-size state tensor are put back.
        rows = self.plan.seq_slot.long()
        kept = {e: t[rows].clone() for e, t in cache.state.items()}
        self._one_step(advance=False)
        for e, t in cache.state.items():
            t[rows] = kept[e]
        self.launches_per_step = ops.LAUNCHES - before + 1
        torch.cuda.synchronize()
        ops.check_status()
        if use_graph:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._one_step(advance=True)

    def _one_step(self, advance: bool) -> None:
        with ops.trace_range("decode step"):
            logits = self.engine.model.forward(self.plan, self.engine.cache)
            ops.sample(logits, self.params, None, self.plan.tokens, fed_pos=self.plan.row_pos)
            if advance:
                ops.advance_rows(self.plan.row_pos, self.plan.row_last)

    def retire(self, row: int) -> None:
        """Row `row` has finished: it stays in the captured batch as a row nobody reads, inside
        its own pages, and `close` records only the tokens it was fed while live."""
        self.live[row] = False

    def _replay(self) -> None:
        for i, (ok, fed, b) in enumerate(zip(self.live, self.fed, self.budgets)):
            if ok and fed >= b:
                raise RuntimeError(f"the loop was sized for {b} tokens of slot {self.slots[i]}")
        if self.graph is not None:
            self.graph.replay()
        else:
            self._one_step(advance=True)
        self.done += 1
        for i, ok in enumerate(self.live):
            if ok:
                self.fed[i] += 1

    def run_device(self, first_tokens, n_steps: int) -> None:
        """`n_steps` steps with the tokens fed back on the device; `first_tokens` (host ids,
        one per sequence) start the loop, None continues from the last produced tokens."""
        if first_tokens is not None:
            self.host_in.copy_(torch.as_tensor(first_tokens, dtype=torch.int32))
            self.plan.tokens.copy_(self.host_in, non_blocking=True)
        for _ in range(n_steps):
            self._replay()

    def step_host(self, tokens) -> list:
        """One step in serving form: token ids in from pinned host memory, new ids back out.
        The id returned for a retired row means nothing."""
        self.host_in.copy_(torch.as_tensor(tokens, dtype=torch.int32))
        self.plan.tokens.copy_(self.host_in, non_blocking=True)
        self._replay()
        self.host_out.copy_(self.plan.tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        if self.done % STATUS_EVERY == 0:
            ops.check_status()
        ids = self.host_out.tolist()
        return ops.check_tokens(ids, self.live)

    def run_host(self, tokens, n_steps: int) -> list:
        for _ in range(n_steps):
            tokens = self.step_host(tokens)
        return tokens

    def close(self) -> None:
        """Tells the cache how far each sequence really got (a windowed group gives back the
        pages it held for the loop); the graph is dropped.  Raises if a kernel of the loop gave
        up on a bounded wait: its tokens are then not to be trusted."""
        cache = self.engine.cache
        for s, at, fed in zip(self.slots, self.start, self.fed):
            if s in cache.records:
                cache.advance(s, at + fed)
        self.start = [at + fed for at, fed in zip(self.start, self.fed)]
        self.fed = [0] * len(self.slots)
        self.done = 0
        self.graph = None
        ops.check_status()
