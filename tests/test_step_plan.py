"""The step's host-side part: validation and the device-side plan's arrays (on the CPU)."""
import pytest
import torch

from sonicboom_b200.cache import Cache, KVNeed
from sonicboom_b200.engine.step import StepEntry, StepError, StepPlan, validate


def cache():
    return Cache([KVNeed(2, 16, 0), KVNeed(2, 16, 70)], [None, None], 64 * 16, torch.float32, "cpu")


def test_plan_arrays():
    c = cache()
    a, b, d = c.open(), c.open(), c.open()
    c.reserve(a, 140); c.advance(a, 140)           # a has history; its window group dropped page 0
    entries = [StepEntry(a, [7], [0]), StepEntry(b, [1, 2, 3], [0, 2]), StepEntry(d, [4, 5], [])]
    for e in entries:
        c.reserve(e.slot, c.length(e.slot) + len(e.tokens))
    p = StepPlan(c, entries, "cpu")
    assert (p.n_rows, p.n_seqs, p.max_new, p.max_len, p.n_want) == (6, 3, 3, 141, 3)
    assert p.tokens.tolist() == [7, 1, 2, 3, 4, 5]
    assert p.row_seq.tolist() == [0, 1, 1, 1, 2, 2]
    assert p.row_pos.tolist() == [140, 0, 1, 2, 0, 1]
    assert p.seq_row0.tolist() == [0, 1, 4, 6] and p.seq_pos0.tolist() == [140, 0, 0]
    assert p.seq_slot.tolist() == [a, b, d]
    assert p.want_rows.tolist() == [0, 1, 3]
    full, win = p.groups
    assert full.page_off.tolist() == [0, 3, 4, 5] and win.page_off.tolist() == [0, 3, 4, 5]
    assert full.page_ids.tolist()[:3] == c.page_list(a, 0) and -1 not in full.page_ids.tolist()
    assert win.page_ids.tolist()[0] == -1 and win.page_ids.tolist()[1] >= 0
    for t in (p.tokens, p.row_seq, p.want_rows, full.page_ids):
        assert t.dtype == torch.int32 and t.data_ptr() % 16 == 0


def test_refusals_before_anything_runs():
    c = cache()
    a = c.open()
    ok = [StepEntry(a, [1, 2], [1])]
    validate(c, ok, vocab=10, max_positions=64)
    for entries, msg in [
            ([], "at least one entry"),
            ([StepEntry(a, [1], []), StepEntry(a, [2], [])], "appears twice"),
            ([StepEntry(5, [1], [])], "holds no sequence"),
            ([StepEntry(a, [], [])], "at least one token"),
            ([StepEntry(a, [1, 10], [])], "token id 10 is outside the vocabulary"),
            ([StepEntry(a, [1, -1], [])], "token id -1"),
            ([StepEntry(a, [1] * 65, [])], "exceed max_position_embeddings"),
            ([StepEntry(a, [1, 2], [2])], "wanted place 2")]:
        with pytest.raises(StepError, match=msg):
            validate(c, entries, vocab=10, max_positions=64)
    assert c.length(a) == 0 and c.page_list(a, 0) == []
