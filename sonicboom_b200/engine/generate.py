"""The generation loop: batches of unequal prompts, stop tokens, sequences that end earlier,
and as many batches one after another as there are requests.

The reference's loop runs one sequence: prefill, first token from the last row's logits, then
one decode step per token until `max_tokens` or a stop (core/src/model/gemma4_plan.cpp:
1631-1637, 1704-1810; capi/src/capi.cpp:2587-3046).  The same loop runs here over a batch:
all prompts in one step, then one token per live sequence per step.  Its decisions are plain
host code over a small engine interface (`open`, `close`, `length`, `step`, `free_pages`,
`free_slots`), so they can be tested without a device.

Rules kept from the reference: a stop token is emitted and then ends its sequence
(core/include/sonicboom/model/plan.h:438-440); the callback gets every token in order and a
non-zero return ends that sequence (capi/include/sonicboom/capi.h:679-682); a request that
cannot fit the context is refused, not wrapped (core/src/model/gemma4_plan.cpp:7334).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional

from ..sampling.params import Sampling


class GenerationError(ValueError):
    pass


@dataclass
class Request:
    prompt: list
    sampling: Sampling
    stop_tokens: frozenset = frozenset()
    index: int = 0


def pages_for(n_tokens: int, page_size: int) -> int:
    return (n_tokens + page_size - 1) // page_size


def form_batch(pending: deque, free_pages: int, free_slots: int, page_size: int,
               max_batch: Optional[int]) -> list:
    """Takes requests from the front of `pending`, in order, while all of them can run to
    their last token together: one slot each, and pages for prompt + max_tokens each."""
    batch, pages = [], 0
    while pending:
        r = pending[0]
        need = pages_for(len(r.prompt) + r.sampling.max_tokens, page_size)
        if batch and (pages + need > free_pages or len(batch) >= free_slots
                      or (max_batch and len(batch) >= max_batch)):
            break
        if not batch and (need > free_pages or free_slots < 1):
            raise GenerationError(
                f"request {r.index} needs {need * page_size} cache tokens "
                f"({len(r.prompt)} prompt + {r.sampling.max_tokens} new), "
                f"the cache has {free_pages * page_size} free")
        batch.append(pending.popleft())
        pages += need
    return batch


def _remaining(r: Request, results: list) -> int:
    return r.sampling.max_tokens - len(results[r.index])


def run_batch(engine, sampler, batch: list, results: list, on_token: Optional[Callable]) -> int:
    """Runs one batch to its end; returns the number of steps it took.  Whatever happens, every
    slot the batch opened has been closed when this returns or raises."""
    held = set()                                 # slots this batch holds

    def release(slot):
        held.discard(slot)
        engine.close(slot)                       # slot and pages are free for the next batch

    try:
        live = []                                # (request, slot, history)
        for r in batch:
            slot = engine.open()
            held.add(slot)
            live.append((r, slot, list(r.prompt)))
        logits = engine.step([(slot, r.prompt, [len(r.prompt) - 1]) for r, slot, _ in live])
        steps = 1
        tokens = sampler.sample(logits, [r.sampling for r, _, _ in live],
                                [engine.length(slot) for _, slot, _ in live], [h for _, _, h in live])
        while True:
            still = []
            for (r, slot, hist), tok in zip(live, tokens):
                out = results[r.index]
                out.append(tok)
                hist.append(tok)
                stop = tok in r.stop_tokens or len(out) >= r.sampling.max_tokens
                if on_token is not None and on_token(r.index, tok):
                    stop = True
                if stop:
                    release(slot)
                else:
                    still.append((r, slot, hist))
            live = still
            if not live:
                return steps
            make_loop = getattr(engine, "decode_loop", None)
            loop = make_loop([slot for _, slot, _ in live], [_remaining(r, results) for r, _, _ in live],
                             [r.sampling for r, _, _ in live]) if make_loop else None
            if loop is not None:
                return steps + _run_device_loop(engine, loop, live, results, on_token, release)
            logits = engine.step([(slot, [hist[-1]], [0]) for _, slot, hist in live])
            steps += 1
            tokens = sampler.sample(logits, [r.sampling for r, _, _ in live],
                                    [engine.length(slot) for _, slot, _ in live], [h for _, _, h in live])
    finally:
        for slot in sorted(held):
            engine.close(slot)


def _run_device_loop(engine, loop, live: list, results: list, on_token: Optional[Callable],
                     release: Callable) -> int:
    """The rest of a batch on the engine's captured decode step: each step's token ids go in
    from the host and the new ids come back.  A finished sequence is retired: it stays in the
    captured batch as a row nobody reads, held inside its own pages by the loop, until fewer
    than half of the rows are live; then the loop is closed, the finished sequences' slots are
    released, and the step is captured again for the live ones with what each of them may still
    produce.  The loop is closed on every way out."""
    steps = 0
    rows = list(live)                            # the captured batch, in row order
    done = [False] * len(rows)
    try:
        while True:
            new = loop.step_host([0 if d else hist[-1] for (_, _, hist), d in zip(rows, done)])
            steps += 1
            for i, ((r, slot, hist), tok) in enumerate(zip(rows, new)):
                if done[i]:
                    continue
                out = results[r.index]
                out.append(tok)
                hist.append(tok)
                stop = tok in r.stop_tokens or len(out) >= r.sampling.max_tokens
                if on_token is not None and on_token(r.index, tok):
                    stop = True
                if stop:
                    done[i] = True
                    loop.retire(i)
            n_live = done.count(False)
            if n_live == 0 or 2 * n_live <= len(rows):
                closing, loop = loop, None
                closing.close()
                for (r, slot, hist), d in zip(rows, done):
                    if d:
                        release(slot)
                rows = [x for x, d in zip(rows, done) if not d]
                if not rows:
                    return steps
                done = [False] * len(rows)
                loop = engine.decode_loop([slot for _, slot, _ in rows],
                                          [_remaining(r, results) for r, _, _ in rows],
                                          [r.sampling for r, _, _ in rows])
    finally:
        if loop is not None:
            loop.close()


def _per_request_stops(stop_tokens, n: int) -> list:
    """None, one collection of ids for every request, or one collection per request."""
    if stop_tokens is None:
        return [frozenset()] * n
    stop_tokens = list(stop_tokens)
    if stop_tokens and all(isinstance(s, (list, tuple, set, frozenset)) for s in stop_tokens):
        return [frozenset(s) for s in stop_tokens]
    return [frozenset(stop_tokens)] * n


def generate(engine, sampler, prompts: list, samplings, stop_tokens=None,
             on_token: Optional[Callable] = None, max_batch: Optional[int] = None,
             max_positions: Optional[int] = None) -> list:
    """Generates for every prompt; returns the new tokens of each, in request order.

    `samplings` is one Sampling for all or one per prompt; `stop_tokens` likewise a set for all
    or one per prompt.  Requests are run in as many batches as the cache needs; a batch runs
    to its end before the next starts, and no request joins a running batch."""
    n = len(prompts)
    if isinstance(samplings, Sampling):
        samplings = [samplings] * n
    if len(samplings) != n:
        raise GenerationError(f"{n} prompts but {len(samplings)} sampling records")
    stop_tokens = _per_request_stops(stop_tokens, n)
    if len(stop_tokens) != n:
        raise GenerationError(f"{n} prompts but {len(stop_tokens)} stop-token sets")
    results = [[] for _ in range(n)]
    pending = deque()
    for i, (p, s, st) in enumerate(zip(prompts, samplings, stop_tokens)):
        s = s.checked()
        if len(p) == 0:
            raise GenerationError(f"request {i}: empty prompt")
        if max_positions is not None and len(p) + s.max_tokens > max_positions:
            raise GenerationError(f"request {i}: {len(p)} prompt + {s.max_tokens} new tokens "
                                  f"exceed the context of {max_positions}")
        if s.max_tokens > 0:
            pending.append(Request(list(p), s, frozenset(st), i))
    while pending:
        batch = form_batch(pending, engine.free_pages(), engine.free_slots(), engine.page_size,
                           max_batch)
        run_batch(engine, sampler, batch, results, on_token)
    return results
