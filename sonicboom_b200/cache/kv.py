"""The cache: a slot for each live sequence, keys and values per schedule entry in pages, and
fixed-size per-sequence state beside them.

Counterpart of the reference's `KvCacheSpec::Layer{kv_heads, head_dim, window}` /
`KvCacheSession` / recurrent `StateSet` (core/include/sonicboom/planner/kv_cache.h:96-170),
rebuilt for batches: the reference gives each conversation a cache set of its own and runs one
at a time; here sequences of a batch share pools of pages.

* A **group** holds the schedule entries with the same need (key/value heads, head size,
  window) and has storage of its own: `[entry, page, k|v, kv head, position in page, hd]`, one
  pool of pages, one page list per sequence (all entries of a group grow together).
* A group with a window gives back the pages whose keys no later query can see, so a
  sequence holds about `window` keys there, however long it grows.
* A **slot** is a sequence's record: its length, its page lists, and its row in every state
  tensor.  Slots and pages are handed back when the sequence ends and are used again; a reused
  slot starts at length 0 with zeroed state, and stale keys in reused pages are never read
  because lengths bound every read.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .pages import CacheError, CacheFull, FreeList

PAGE_SIZE = 64


@dataclass(frozen=True)
class KVNeed:
    """What a mixer asks of the cache for one schedule entry."""
    n_kv_heads: int
    head_dim: int
    window: int = 0            # 0: all keys stay; n: only the last n keys are ever read


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-sequence state a part asks for: one tensor row per slot."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class CacheGroup:
    def __init__(self, need: KVNeed, entries: list[int], n_pages: int, page_size: int, dtype,
                 device):
        self.need, self.entries, self.page_size = need, list(entries), page_size
        self.pool = FreeList(n_pages, "page")
        # zeroed once: a page's unused tail is multiplied by zero probabilities, so it must
        # never hold NaN or infinity bit patterns; what sequences write later is finite
        self.storage = torch.zeros((len(entries), n_pages, 2, need.n_kv_heads, page_size,
                                    need.head_dim), dtype=dtype, device=device)
        self._index = {e: i for i, e in enumerate(entries)}

    def entry_storage(self, entry: int) -> torch.Tensor:
        """[page, k|v, kv head, position in page, hd] of one schedule entry."""
        return self.storage[self._index[entry]]

    def bytes_per_token(self) -> int:
        n = self.need
        return len(self.entries) * 2 * n.n_kv_heads * n.head_dim * self.storage.element_size()


@dataclass
class SlotRecord:
    slot: int
    length: int = 0
    pages: list = field(default_factory=list)     # per group: list of page ids, None = given back


class Cache:
    """All groups, the slot table and the state tensors of one engine."""

    def __init__(self, kv_needs: list, state_needs: list, max_tokens: int, dtype, device,
                 n_slots: Optional[int] = None, page_size: int = PAGE_SIZE):
        """`kv_needs[i]` / `state_needs[i]` are what schedule entry i asks for (None: nothing).
        `max_tokens` is the most tokens live sequences hold together, each sequence's count
        rounded up to a whole page."""
        if max_tokens <= 0:
            raise CacheError(f"max_tokens = {max_tokens}")
        self.page_size = page_size
        self.n_pages = (max_tokens + page_size - 1) // page_size
        self.n_slots = int(n_slots) if n_slots else min(self.n_pages, 4096)
        self.dtype, self.device = dtype, torch.device(device)
        self.slots = FreeList(self.n_slots, "slot")
        self.records: dict[int, SlotRecord] = {}
        by_need: dict[KVNeed, list[int]] = {}
        for entry, need in enumerate(kv_needs):
            if need is not None:
                by_need.setdefault(need, []).append(entry)
        self.groups = [CacheGroup(need, entries, self.n_pages, page_size, dtype, device)
                       for need, entries in by_need.items()]
        self.group_of_entry = {e: gi for gi, g in enumerate(self.groups) for e in g.entries}
        self.state = {entry: torch.zeros((self.n_slots, *need.shape), dtype=need.dtype, device=device)
                      for entry, need in enumerate(state_needs) if need is not None}

    # ------------------------------------------------------------------ sequences
    def open(self) -> int:
        """Takes a slot for a new sequence: length 0, no pages, zeroed state."""
        (slot,) = self.slots.take(1)
        self.records[slot] = SlotRecord(slot, 0, [[] for _ in self.groups])
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def length(self, slot: int) -> int:
        return self._record(slot).length

    def _record(self, slot: int) -> SlotRecord:
        if slot not in self.records:
            raise CacheError(f"slot {slot} holds no sequence")
        return self.records[slot]

    def pages_needed(self, slot: int, new_len: int) -> int:
        """Pages one group has to add so that the sequence can reach `new_len`."""
        rec = self._record(slot)
        have = len(rec.pages[0]) if self.groups else 0
        return max(0, (new_len + self.page_size - 1) // self.page_size - have)

    def reserve(self, slot: int, new_len: int) -> None:
        """Adds pages in every group so that positions up to new_len-1 can be written.
        Nothing changes when any group cannot supply them (raises CacheFull)."""
        rec = self._record(slot)
        if new_len < rec.length:
            raise CacheError(f"slot {slot}: cannot shrink from {rec.length} to {new_len}")
        want = (new_len + self.page_size - 1) // self.page_size
        adds = [want - len(p) for p in rec.pages]
        for g, add in zip(self.groups, adds):
            if add > g.pool.free_count:
                raise CacheFull(f"slot {slot} needs {add} more page(s) of {self.page_size} tokens, "
                                f"{g.pool.free_count} of {g.pool.n} are free")
        for g, pages, add in zip(self.groups, rec.pages, adds):
            if add > 0:
                pages.extend(g.pool.take(add))

    def reserve_many(self, wants) -> None:
        """`reserve` for several sequences at once, `wants` being (slot, new_len) pairs: either
        every one of them gets its pages or nothing changes (raises CacheFull)."""
        wants = list(wants)
        need = [0] * len(self.groups)
        for slot, new_len in wants:
            rec = self._record(slot)
            if new_len < rec.length:
                raise CacheError(f"slot {slot}: cannot shrink from {rec.length} to {new_len}")
            want = (new_len + self.page_size - 1) // self.page_size
            for gi, pages in enumerate(rec.pages):
                need[gi] += max(0, want - len(pages))
        for g, n in zip(self.groups, need):
            if n > g.pool.free_count:
                raise CacheFull(f"{len(wants)} sequences need {n} more page(s) of {self.page_size} "
                                f"tokens together, {g.pool.free_count} of {g.pool.n} are free")
        for slot, new_len in wants:
            self.reserve(slot, new_len)

    def advance(self, slot: int, new_len: int) -> None:
        """Records the new length after a step and gives back pages a window has left behind."""
        rec = self._record(slot)
        if new_len < rec.length or any(len(p) * self.page_size < new_len for p in rec.pages):
            raise CacheError(f"slot {slot}: advance to {new_len} without pages for it")
        rec.length = new_len
        for g, pages in zip(self.groups, rec.pages):
            w = g.need.window
            if w <= 0:
                continue
            # the next query sits at position >= new_len and sees keys j > position - w
            dead_pages = max(0, new_len - w + 1) // self.page_size     # pages wholly at j <= new_len - w
            give = [pages[i] for i in range(min(dead_pages, len(pages))) if pages[i] is not None]
            if give:
                g.pool.give_back(give)
                for i in range(min(dead_pages, len(pages))):
                    pages[i] = None

    def truncate(self, slot: int, new_len: int) -> bool:
        """Cuts a sequence back to its first `new_len` tokens (prefix reuse).  Returns False,
        changing nothing, when a windowed group has already given back pages that the shorter
        sequence would read again, or when the model keeps fixed-size state per sequence (it
        was advanced by the tokens that would be cut)."""
        rec = self._record(slot)
        if not 0 <= new_len <= rec.length:
            raise CacheError(f"slot {slot}: cannot truncate from {rec.length} to {new_len}")
        if self.state and new_len < rec.length:
            return False         # fixed-size state has moved on with the tokens and cannot go back
        keep = (new_len + self.page_size - 1) // self.page_size
        for g, pages in zip(self.groups, rec.pages):
            first_seen = max(0, new_len - g.need.window + 1) // self.page_size if g.need.window else 0
            if any(p is None for p in pages[first_seen:keep]):
                return False
        for g, pages in zip(self.groups, rec.pages):
            g.pool.give_back([p for p in pages[keep:] if p is not None])
            del pages[keep:]
        rec.length = new_len
        return True

    def close(self, slot: int) -> None:
        """Ends a sequence: its pages and its slot go back to the pools."""
        rec = self._record(slot)
        for g, pages in zip(self.groups, rec.pages):
            g.pool.give_back([p for p in pages if p is not None])
        del self.records[slot]
        self.slots.give_back([slot])

    def page_list(self, slot: int, group: int) -> list[int]:
        """Page ids of a sequence in one group, -1 where a page was given back."""
        return [-1 if p is None else p for p in self._record(slot).pages[group]]

    # ------------------------------------------------------------------ accounting
    def tokens_held(self) -> int:
        """Tokens live sequences hold, each rounded up to a whole page."""
        ps = self.page_size
        return sum((r.length + ps - 1) // ps * ps for r in self.records.values())

    def check(self) -> None:
        """Every slot and page is free or held by exactly one sequence."""
        self.slots.check()
        if set(self.records) != {s for s in range(self.n_slots) if self.slots.is_held(s)}:
            raise CacheError("slot table and sequence records disagree")
        for gi, g in enumerate(self.groups):
            g.pool.check()
            owned = [p for r in self.records.values() for p in r.pages[gi] if p is not None]
            if len(owned) != len(set(owned)):
                raise CacheError(f"group {gi}: a page is held by two sequences")
            if len(owned) != g.pool.held_count:
                raise CacheError(f"group {gi}: {g.pool.held_count} pages out, sequences hold {len(owned)}")
