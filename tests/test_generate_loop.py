"""The generation loop's decisions, with a fake engine and sampler (no device)."""
from collections import deque

import pytest

from sonicboom_b200.engine.generate import (GenerationError, Request, form_batch, generate,
                                            pages_for)
from sonicboom_b200.sampling import Sampling


class FakeEngine:
    """Counts instead of computing: 'logits' are (slot, tokens fed so far) per wanted row."""
    page_size = 64

    def __init__(self, n_pages=8, n_slots=4):
        self.n_pages, self.n_slots = n_pages, n_slots
        self.lengths, self.fed, self.steps, self.opened = {}, {}, [], []

    def open(self):
        slot = min(set(range(self.n_slots)) - set(self.lengths))
        self.lengths[slot], self.fed[slot] = 0, []
        self.opened.append(slot)
        return slot

    def close(self, slot):
        del self.lengths[slot], self.fed[slot]

    def length(self, slot):
        return self.lengths[slot]

    def free_pages(self):
        return self.n_pages - sum(pages_for(n, 64) for n in self.lengths.values())

    def free_slots(self):
        return self.n_slots - len(self.lengths)

    def step(self, entries):
        self.steps.append([(s, list(t)) for s, t, _ in entries])
        out = []
        for slot, tokens, want in entries:
            assert slot in self.lengths and len(want) == 1 and want[0] == len(tokens) - 1
            self.fed[slot] += tokens
            self.lengths[slot] += len(tokens)
            assert pages_for(self.lengths[slot], 64) <= self.n_pages
            out.append(list(self.fed[slot]))
        return out


class FakeSampler:
    """Next token = (sum of the sequence so far) % 50; records what it was asked."""

    def __init__(self):
        self.calls = []

    def sample(self, logits, samplings, positions, histories):
        self.calls.append((positions, [list(h) for h in histories]))
        for fed, pos, hist in zip(logits, positions, histories):
            assert fed == hist and pos == len(hist)     # position of the token being produced
        return [sum(h) % 50 for h in histories]


def expected(prompt, n, stops=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = sum(seq) % 50
        out.append(t); seq.append(t)
        if t in stops:
            break
    return out


def test_batch_of_unequal_prompts_each_as_if_alone():
    eng, smp = FakeEngine(), FakeSampler()
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9]]
    out = generate(eng, smp, prompts, Sampling(max_tokens=6))
    assert out == [expected(p, 6) for p in prompts]
    assert len(eng.steps) == 6 and [len(s) for s in eng.steps] == [3] * 6
    assert eng.steps[0] == [(0, [1, 2, 3]), (1, [4]), (2, [5, 6, 7, 8, 9])]   # prompts: one step
    assert all(len(t) == 1 for s in eng.steps[1:] for _, t in s)             # then one token each
    assert not eng.lengths                                                   # all slots returned


def test_sequences_end_earlier_and_leave_the_batch():
    eng, smp = FakeEngine(), FakeSampler()
    prompts = [[1, 2, 3], [4], [5, 6, 7]]
    per = [Sampling(max_tokens=2), Sampling(max_tokens=7), Sampling(max_tokens=4)]
    out = generate(eng, smp, prompts, per)
    assert [len(o) for o in out] == [2, 7, 4]
    assert out == [expected(p, s.max_tokens) for p, s in zip(prompts, per)]
    assert [len(s) for s in eng.steps] == [3, 3, 2, 2, 1, 1, 1]


def test_stop_token_is_emitted_then_ends_the_sequence():
    eng, smp = FakeEngine(), FakeSampler()
    prompts = [[1, 2, 3], [10, 11]]
    free = [expected(p, 8) for p in prompts]
    stop = free[0][2]
    out = generate(eng, smp, prompts, Sampling(max_tokens=8), stop_tokens=[[stop], []])
    assert out[0] == free[0][:3] and out[0][-1] == stop and out[1] == free[1]
    out2 = generate(FakeEngine(), FakeSampler(), prompts, Sampling(max_tokens=8), stop_tokens=[stop])
    assert out2[0] == free[0][:3]
    assert out2[1] == expected(prompts[1], 8, stops=[stop])


def test_callback_gets_tokens_in_order_and_can_stop():
    seen = []

    def cb(i, tok):
        seen.append((i, tok))
        return i == 1 and len([1 for j, _ in seen if j == 1]) == 2
    out = generate(FakeEngine(), FakeSampler(), [[1], [2], [3]], Sampling(max_tokens=4), on_token=cb)
    assert [len(o) for o in out] == [4, 2, 4]
    assert [t for i, t in seen if i == 0] == out[0]


def test_more_requests_than_the_cache_holds_run_as_batches_and_reuse_slots():
    eng, smp = FakeEngine(n_pages=4, n_slots=2), FakeSampler()
    prompts = [[i + 1] * (10 + 30 * i) for i in range(5)]       # 10..130 tokens
    out = generate(eng, smp, prompts, Sampling(max_tokens=5))
    assert out == [expected(p, 5) for p in prompts]
    first_steps = [s for s in eng.steps if any(len(t) > 1 for _, t in s)]
    assert len(first_steps) >= 3                                 # several batches, one after another
    assert set(eng.opened) == {0, 1} and len(eng.opened) == 5    # two slots served five requests
    assert not eng.lengths
    # no request joins a running batch: every multi-token step holds only fresh sequences
    for s in first_steps:
        assert all(len(t) > 1 for _, t in s)


def test_form_batch_rules():
    def reqs(*sizes):
        return deque(Request([0] * p, Sampling(max_tokens=n), frozenset(), i)
                     for i, (p, n) in enumerate(sizes))
    q = reqs((60, 4), (60, 5), (10, 10))
    b = form_batch(q, free_pages=3, free_slots=8, page_size=64, max_batch=None)
    assert [r.index for r in b] == [0, 1] and len(q) == 1        # 1 + 2 pages fit, the third does not
    q = reqs((10, 1), (10, 1), (10, 1))
    assert len(form_batch(q, 100, 2, 64, None)) == 2             # slots bound it
    q = reqs((10, 1), (10, 1), (10, 1))
    assert len(form_batch(q, 100, 8, 64, max_batch=1)) == 1
    with pytest.raises(GenerationError, match="request 0 needs 192 cache tokens"):
        form_batch(reqs((130, 10)), 2, 8, 64, None)


def test_refusals():
    eng, smp = FakeEngine(), FakeSampler()
    with pytest.raises(GenerationError, match="empty prompt"):
        generate(eng, smp, [[1], []], Sampling(max_tokens=2))
    with pytest.raises(GenerationError, match="exceed the context"):
        generate(eng, smp, [[1] * 10], Sampling(max_tokens=7), max_positions=16)
    with pytest.raises(GenerationError, match="sampling records"):
        generate(eng, smp, [[1], [2]], [Sampling()])
    with pytest.raises(ValueError, match="sampling.top_p"):
        generate(eng, smp, [[1]], Sampling(top_p=1.5))
    assert generate(eng, smp, [[1], [2]], Sampling(max_tokens=0)) == [[], []]
    assert not eng.steps


def test_sampling_record_checks():
    s = Sampling().checked()
    assert s.temperature == 0.0 and s.top_k == 0 and s.top_p == 1.0 and s.repeat_last_n == 64
    assert not s.penalizes
    assert Sampling(repeat_penalty=0.0).checked().repeat_penalty == 1.0      # 0 means off
    assert Sampling(repeat_penalty=1.3).checked().penalizes
    assert not Sampling(repeat_penalty=1.3, repeat_last_n=0).checked().penalizes
    for field, value in [("temperature", -0.1), ("top_k", -1), ("min_p", 2.0), ("seed", 2 ** 64),
                         ("repeat_last_n", 5000), ("repeat_penalty", -1.0), ("max_tokens", 1.5),
                         ("temperature", float("nan"))]:
        with pytest.raises(ValueError, match=f"sampling.{field}"):
            Sampling(**{field: value}).checked()


def test_packed_sampler_records():
    import numpy as np
    from sonicboom_b200.sampling.sampler import _RECORD, pack_params
    a = Sampling(temperature=0.7, top_k=5, seed=2 ** 40 + 3, repeat_penalty=1.2, repeat_last_n=3).checked()
    b = Sampling().checked()
    rec, hist = pack_params([a, b], [17, 4], [[1, 2, 3, 4, 5], [9, 9]])
    r = rec.view(_RECORD)
    assert r["seed"][0] == 2 ** 40 + 3 and r["position"].tolist() == [17, 4]
    assert r["history_len"].tolist() == [3, 0] and r["top_k"].tolist() == [5, 0]
    assert hist.tolist() == [[3, 4, 5], [-1, -1, -1]]
    assert abs(float(r["temperature"][0]) - 0.7) < 1e-6
    rec, hist = pack_params([b], [0], [[1, 2]])
    assert hist is None


def test_a_row_without_a_sampled_token_is_an_error():
    """The device sampler writes -1 where no candidate survives (logits that are not finite);
    wherever ids are read on the host that becomes an error that names the row."""
    from sonicboom_b200 import ops
    assert ops.check_tokens([3, 0, 7]) == [3, 0, 7]
    with pytest.raises(ops.KernelError, match="row 1"):
        ops.check_tokens([3, -1, 7])


# ------------------------------------------------------------------ the captured decode loop
class FakeLoop:
    """Stands in for engine.decode.DecodeLoop with the same contract: per-row budgets and
    reservations, positions that advance as the device kernel advances them (one step at a
    time, never past the last reserved position), `retire`, and `close` recording what each
    row was fed while live."""

    def __init__(self, engine, slots, budgets, samplings):
        assert len(slots) == len(budgets) == len(samplings) and min(budgets) >= 1
        self.engine, self.slots, self.budgets = engine, list(slots), list(budgets)
        self.start = [engine.lengths[s] for s in slots]
        for s, at, b in zip(slots, self.start, budgets):
            engine.reserved[s] = max(engine.reserved.get(s, 0), pages_for(at + b, 64))
        assert engine.pages_out() <= engine.n_pages, "the loop reserved more than the cache holds"
        self.pos = list(self.start)
        self.last = [at + b - 1 for at, b in zip(self.start, budgets)]
        self.live, self.fed, self.closed = [True] * len(slots), [0] * len(slots), False
        self.positions_written = [[] for _ in slots]
        engine.loops.append(self)

    def retire(self, row):
        assert self.live[row]
        self.live[row] = False

    def step_host(self, tokens):
        assert not self.closed
        out = []
        for i, (slot, tok) in enumerate(zip(self.slots, tokens)):
            # every row of the captured batch runs, live or not, and writes at its position
            assert self.pos[i] <= self.last[i] < self.engine.reserved[slot] * 64
            self.positions_written[i].append(self.pos[i])
            if self.live[i]:
                assert self.fed[i] < self.budgets[i], "a live row was stepped past its budget"
                assert self.pos[i] == self.start[i] + self.fed[i]
                self.engine.fed[slot].append(tok)
                self.fed[i] += 1
                out.append(sum(self.engine.fed[slot]) % 50)
            else:
                out.append(-1)                   # a retired row's id means nothing
            self.pos[i] = min(self.pos[i] + 1, self.last[i])
        self.engine.loop_steps.append(len(self.slots))
        return out

    def close(self):
        assert not self.closed, "a loop was closed twice"
        self.closed = True
        for slot, at, fed in zip(self.slots, self.start, self.fed):
            if slot in self.engine.lengths:
                self.engine.lengths[slot] = at + fed


class LoopEngine(FakeEngine):
    """FakeEngine with a captured decode loop; pages are counted as the real cache counts them
    (what a sequence holds or has reserved), and slots must be closed exactly once."""

    def __init__(self, n_pages=64, n_slots=8):
        super().__init__(n_pages, n_slots)
        self.reserved, self.loops, self.loop_steps, self.closed_slots = {}, [], [], []

    def pages_out(self):
        return sum(max(pages_for(n, 64), self.reserved.get(s, 0)) for s, n in self.lengths.items())

    def free_pages(self):
        return self.n_pages - self.pages_out()

    def close(self, slot):
        assert slot in self.lengths, f"slot {slot} closed twice"
        self.closed_slots.append(slot)
        self.reserved.pop(slot, None)
        super().close(slot)

    def decode_loop(self, slots, budgets, samplings):
        return FakeLoop(self, slots, budgets, samplings)


def check_loops(eng):
    assert not eng.lengths and sorted(eng.closed_slots) == sorted(eng.opened)   # each slot once
    assert all(l.closed for l in eng.loops)
    for l in eng.loops:
        for written, last in zip(l.positions_written, l.last):
            assert max(written) <= last


def test_device_loop_with_per_request_budgets_in_batches_of_three_to_seven():
    for n in range(3, 8):
        eng, smp = LoopEngine(), FakeSampler()
        prompts = [[i + 1] * (1 + 9 * i) for i in range(n)]
        per = [Sampling(max_tokens=2 + 3 * ((i * 5) % 7)) for i in range(n)]
        out = generate(eng, smp, prompts, per)
        assert out == [expected(p, s.max_tokens) for p, s in zip(prompts, per)], n
        check_loops(eng)
        # the step is captured again once half of the rows (or more) have finished: never
        # does a loop keep running with more than half of its rows retired
        sizes = [len(l.slots) for l in eng.loops]
        assert sizes[0] == n and all(2 * b <= a or b < a for a, b in zip(sizes, sizes[1:]))
        assert len(eng.loops) >= 2


def test_device_loop_recaptures_at_half():
    eng, smp = LoopEngine(), FakeSampler()
    prompts = [[1], [2], [3], [4]]
    per = [Sampling(max_tokens=m) for m in (3, 9, 4, 9)]
    out = generate(eng, smp, prompts, per)
    assert [len(o) for o in out] == [3, 9, 4, 9]
    check_loops(eng)
    # first token from the prompt step; row 0 ends after 2 loop steps (3 of 4 live: no
    # recapture), row 2 after 3 (2 of 4 live: recapture with the two live rows)
    assert [len(l.slots) for l in eng.loops] == [4, 2]
    assert eng.loop_steps == [4, 4, 4] + [2] * 5
    assert eng.loops[0].fed == [2, 3, 3, 3] and eng.loops[1].budgets == [5, 5]


def test_device_loop_stop_tokens_and_callback():
    prompts = [[1, 2, 3], [10, 11], [7], [9, 9], [4, 4, 4]]
    free = [expected(p, 12) for p in prompts]
    stop = free[0][4]
    eng = LoopEngine()
    seen = []

    def cb(i, tok):
        seen.append((i, tok))
        return i == 3 and sum(1 for j, _ in seen if j == 3) == 6
    out = generate(eng, FakeSampler(), prompts, Sampling(max_tokens=12),
                   stop_tokens=[[stop], [], [], [], []], on_token=cb)
    assert out[0] == free[0][:5] and out[3] == free[3][:6]
    assert out[1] == free[1] and out[2] == free[2] and out[4] == free[4]
    assert [t for i, t in seen if i == 1] == out[1]
    check_loops(eng)


def test_device_loop_at_exactly_the_cache_form_batch_budgets():
    """Two requests of 10 prompt tokens, one allowed 10 new tokens and one 1,000: 1 + 16 pages.
    A loop that reserved the largest budget for every row would need 32."""
    eng = LoopEngine(n_pages=17, n_slots=2)
    prompts = [[1] * 10, [2] * 10]
    per = [Sampling(max_tokens=10), Sampling(max_tokens=1000)]
    out = generate(eng, FakeSampler(), prompts, per)
    assert [len(o) for o in out] == [10, 1000] and out[0] == expected(prompts[0], 10)
    check_loops(eng)
    assert len(eng.opened) == 2 and len(set(eng.opened)) == 2        # one batch


def test_slots_are_closed_when_a_step_fails():
    class Boom(RuntimeError):
        pass

    class FailingLoop(FakeLoop):
        def step_host(self, tokens):
            if len(self.engine.loop_steps) == 2:
                raise Boom("a kernel gave up")
            return super().step_host(tokens)

    class FailingEngine(LoopEngine):
        def decode_loop(self, slots, budgets, samplings):
            return FailingLoop(self, slots, budgets, samplings)

    eng = FailingEngine()
    with pytest.raises(Boom):
        generate(eng, FakeSampler(), [[1], [2], [3]], Sampling(max_tokens=8))
    assert not eng.lengths and sorted(eng.closed_slots) == sorted(eng.opened)
    assert all(l.closed for l in eng.loops)

    class FullEngine(LoopEngine):
        def decode_loop(self, slots, budgets, samplings):
            from sonicboom_b200.cache import CacheFull
            raise CacheFull("no pages")
    eng = FullEngine()
    with pytest.raises(Exception, match="no pages"):
        generate(eng, FakeSampler(), [[1], [2]], Sampling(max_tokens=8))
    assert not eng.lengths and sorted(eng.closed_slots) == sorted(eng.opened)
