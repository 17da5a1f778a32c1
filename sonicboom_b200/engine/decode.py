"""The decode loop on the device: one captured CUDA graph per batch, replayed once a token.

The reference captures its decode step as a CUDA graph and replays it per token, feeding each
argmax back through device memory (`greedy_step`: set the position, one cudaGraphLaunch, read
the token; core/src/model/gemma4_plan.cpp:1650-1696, core/include/sonicboom/hal/command.h:
34-45).  The same is done here for a batch: the step's plan lives in persistent device
buffers; the graph runs the model's own step (the same parts and kernels as an eager step),
the sampler, which writes the new tokens where the next step's embedding reads them, and a
one-line kernel that advances the positions.  Pages for all tokens the loop may produce are
reserved up front, so the page tables in the graph stay valid.

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

    def __init__(self, cache, slots, device):
        n = len(slots)
        lengths = [cache.length(s) for s in slots]
        self.n_rows = self.n_seqs = self.n_want = n
        self.max_new = 1
        ar = torch.arange(n + 1, dtype=torch.int32)
        self.tokens = torch.zeros(n, dtype=torch.int32, device=device)
        self.row_seq = ar[:n].to(device)
        self.row_pos = torch.tensor(lengths, dtype=torch.int32, device=device)
        self.seq_row0 = ar.to(device)
        self.seq_pos0 = self.row_pos                       # one new row per sequence
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=device)
        self.want_rows = self.row_seq
        self.groups = []
        for gi in range(len(cache.groups)):
            lists = [cache.page_list(s, gi) for s in slots]
            off = np.zeros(n + 1, dtype=np.int32)
            off[1:] = np.cumsum([len(l) for l in lists])
            ids = np.asarray([p for l in lists for p in l], dtype=np.int32)
            self.groups.append(GroupPlan(torch.from_numpy(off).to(device),
                                         torch.from_numpy(ids).to(device), cache.page_size))
        self.max_len = max(len(l) for l in lists) * cache.page_size if cache.groups else 0
        self._scratch = None

    def scratch(self, nbytes: int, device):
        if nbytes <= 0:
            return None
        if self._scratch is None or self._scratch.numel() < nbytes:
            self._scratch = torch.empty(nbytes, dtype=torch.uint8, device=device)
        return self._scratch


class DecodeLoop:
    def __init__(self, engine, slots, max_new: int, samplings=None, use_graph: bool = True):
        """`slots`: live sequences that have been prefilled; `max_new`: the most tokens the
        loop will be asked to produce for any of them."""
        cache, model = engine.cache, engine.model
        if any(g.need.window > 0 for g in cache.groups):
            raise ValueError("the device decode loop needs page tables that do not change; "
                             "a windowed cache group gives pages back as it goes")
        self.engine, self.slots, self.device = engine, list(slots), model.device
        n = len(self.slots)
        self.max_new, self.done = int(max_new), 0
        for s in self.slots:
            cache.reserve(s, min(cache.length(s) + self.max_new, model.spec.max_positions))
        self.plan = DecodePlan(cache, self.slots, self.device)
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
        # one eager run first: builds what is built lazily and sets kernel attributes; it writes
        # keys and values at the current positions, which the first real step overwrites
        self._one_step(advance=False)
        self.launches_per_step = ops.LAUNCHES - before + 1
        torch.cuda.synchronize()
        if use_graph:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._one_step(advance=True)

    def _one_step(self, advance: bool) -> None:
        logits = self.engine.model.forward(self.plan, self.engine.cache)
        ops.sample(logits, self.params, None, self.plan.tokens, fed_pos=self.plan.row_pos)
        if advance:
            ops.add_i32(self.plan.row_pos, 1)

    def _replay(self) -> None:
        if self.done >= self.max_new:
            raise RuntimeError(f"the loop was sized for {self.max_new} tokens")
        if self.graph is not None:
            self.graph.replay()
        else:
            self._one_step(advance=True)
        self.done += 1

    def run_device(self, first_tokens, n_steps: int) -> None:
        """`n_steps` steps with the tokens fed back on the device; `first_tokens` (host ids,
        one per sequence) start the loop, None continues from the last produced tokens."""
        if first_tokens is not None:
            self.host_in.copy_(torch.as_tensor(first_tokens, dtype=torch.int32))
            self.plan.tokens.copy_(self.host_in, non_blocking=True)
        for _ in range(n_steps):
            self._replay()

    def step_host(self, tokens) -> list:
        """One step in serving form: token ids in from pinned host memory, new ids back out."""
        self.host_in.copy_(torch.as_tensor(tokens, dtype=torch.int32))
        self.plan.tokens.copy_(self.host_in, non_blocking=True)
        self._replay()
        self.host_out.copy_(self.plan.tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return ops.check_tokens(self.host_out.tolist())

    def run_host(self, tokens, n_steps: int) -> list:
        for _ in range(n_steps):
            tokens = self.step_host(tokens)
        return tokens

    def close(self) -> None:
        """Tells the cache how far the sequences got; the graph is dropped."""
        cache = self.engine.cache
        for s in self.slots:
            if s in cache.records:
                cache.advance(s, cache.length(s) + self.done)
        self.done = 0
        self.graph = None
