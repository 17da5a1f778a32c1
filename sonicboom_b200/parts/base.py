"""Interfaces of the parts a layer is put together from, and the registries that name them.

A part knows its own sizes and constants (they come in through its spec record) and nothing
about the model it sits in.  The configuration chooses parts layer by layer through the
`kind` strings of the spec records; `register_*` adds a kind without touching this package.

Every part follows the same life cycle:
    part = Kind(spec, dtype, device)      # sizes and constants only
    part.tensor_requests()                # which tensors it wants, by name and shape
    part.bind(get)                        # get(name) -> device tensor; fuse / lay out weights
    part.forward(...)                     # run on the rows of one step

What a step hands to parts is a `StepContext`: the step's device-side plan (rows, positions,
page tables), the cache, and which schedule entry is running.

A norm that directly follows a part's last product can be computed by the kernel that finishes
the product.  Whoever will apply the norm names it in `ctx.next_norm` before it calls the part;
a part that ends in a product calls `ctx.linear(...)` instead of `ops.linear(...)`, which hands
the normed rows back through `ctx.take_normed(norm, rows)`.  Across blocks the model names the
next entry's first norm in `ctx.after_block_norm`, and a block whose result is its last part's
result passes it on as that part's `next_norm`.  Parts and blocks that ignore all this are still
right: `take_normed` then returns None and the caller runs the norm itself.

`ctx.next_weights` is a hint of the same kind: weights that something after the running part
streams and cannot request early itself (`first_weights(rows)` of a part or block says which).
`ctx.linear` passes it to the product kernel, whose blocks ask for it into L2 as they end.  A
hint changes no result, and ignoring it costs nothing.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from .. import ops
from ..cache.kv import Cache, KVNeed, StateNeed
from ..weights.loader import TensorRequest


@dataclass
class StepContext:
    plan: object                   # engine.step.StepPlan
    cache: Cache
    entry: int = 0                 # index of the running schedule entry
    kv_entry: int = 0              # entry whose cache is read (== entry when it owns one)
    owns_cache: bool = True
    next_norm: Optional["Norm"] = None     # the norm the caller applies to the running part's result
    after_block_norm: Optional["Norm"] = None   # the first norm of the entry that runs next (for blocks)
    next_weights: Optional[torch.Tensor] = None         # an L2 hint for the running part's last product
    after_block_weights: Optional[torch.Tensor] = None  # what the entry that runs next streams first, if it asks late
    _normed: Optional[tuple] = None        # (norm, rows, normed rows) of the last `linear` that had one

    def linear(self, a, w, out, epilogue, residual=None, bias=None, act_dtype=None):
        """ops.linear into float32 `out`; when `next_norm` is an RMS norm with a plain weight,
        its result over the finished rows (in `act_dtype`) is produced with it and kept for
        `take_normed`."""
        norm, self.next_norm, self._normed = self.next_norm, None, None
        warm, self.next_weights = self.next_weights, None
        rms = norm.as_rms() if norm is not None else None
        if rms is None or out.dtype != torch.float32 or epilogue == ops.EPI_SWIGLU:
            return ops.linear(a, w, out, epilogue, bias=bias, residual=residual, warm=warm)
        normed = torch.empty(out.shape, dtype=act_dtype or a.dtype, device=out.device)
        ops.linear(a, w, out, epilogue, bias=bias, residual=residual, norm=(rms[0], rms[1], normed),
                   warm=warm)
        self._normed = (norm, out, normed)
        return out

    def take_normed(self, norm, x) -> Optional[torch.Tensor]:
        """`norm` of the rows `x`, if the part that just ran left it behind; else None."""
        kept, self._normed, self.next_norm = self._normed, None, None
        return kept[2] if kept is not None and kept[0] is norm and kept[1] is x else None

    def kv_storage(self) -> torch.Tensor:
        """[page, k|v, kv head, position in page, hd] of the cache this entry reads."""
        g = self.cache.groups[self.cache.group_of_entry[self.kv_entry]]
        return g.entry_storage(self.kv_entry)

    def kv_group(self) -> int:
        return self.cache.group_of_entry[self.kv_entry]

    def state(self) -> torch.Tensor:
        """[slot, ...] state tensor of the running entry; rows are `plan.seq_slot`."""
        return self.cache.state[self.entry]


class Part:
    def tensor_requests(self) -> list[TensorRequest]:
        return []

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        pass


class Norm(Part):
    """forward(x float32 [rows, width], out_dtype, rows=None) -> [n, width] in out_dtype;
    with `rows` (device int32) only those rows of x are normed, in that order."""

    def forward(self, x, out_dtype, rows=None):
        raise NotImplementedError

    def as_rms(self) -> Optional[tuple]:
        """(weight, eps) when the norm is y = x / sqrt(mean(x^2) + eps) * weight, else None:
        what a product kernel needs to apply it to its own result."""
        return None


class PositionEncoding(Part):
    """Supplies what the rotation kernel consumes: `rotary_dim` and a float32 table
    `inv_freq[rotary_dim/2]` on the device (angle = position * inv_freq[i])."""
    rotary_dim: int = 0
    inv_freq: Optional[torch.Tensor] = None


class Mixer(Part):
    """forward(h [rows, width] in the activation dtype, ctx, residual=None) -> float32
    [rows, width]: the mixed rows, plus `residual` (which it may overwrite) when given."""

    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, h, ctx: StepContext, residual=None):
        raise NotImplementedError

    def first_weights(self, rows: int) -> Optional[torch.Tensor]:
        """The weights its forward streams first, if at `rows` rows they are worth an L2 hint
        from whatever runs before it (`ops.requests_weights_late`); else None."""
        return None


class FeedForward(Part):
    """forward(h [rows, width], ctx, residual=None) -> float32 [rows, width]."""

    def forward(self, h, ctx: StepContext, residual=None):
        raise NotImplementedError


class Block(Part):
    """forward(x float32 [rows, width], ctx) -> float32 [rows, width] (may be x itself)."""

    def forward(self, x, ctx: StepContext):
        raise NotImplementedError

    def input_norm(self) -> Optional[Norm]:
        """The norm this arrangement applies to its input first, if it starts with one: the
        entry before it may then deliver the normed rows (see `StepContext.take_normed`)."""
        return None

    def first_weights(self, rows: int) -> Optional[torch.Tensor]:
        """As `Mixer.first_weights`, for the block's first product."""
        return None

    def kv_need(self):
        return None

    def state_need(self):
        return None


NORMS: dict[str, type] = {}
POSITION_ENCODINGS: dict[str, type] = {}
MIXERS: dict[str, type] = {}
FEED_FORWARDS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}


def _register(table, what):
    def register(kind: str, cls=None):
        def put(c):
            table[kind] = c
            return c
        return put(cls) if cls is not None else put
    register.__doc__ = f"Registers a {what} class under a `kind` name (usable as a decorator)."
    return register


register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_block = _register(BLOCKS, "block arrangement")


def make(table: dict, what: str, spec, dtype, device):
    from ..config.specs import ConfigError
    if spec.kind not in table:
        raise ConfigError(f"unknown {what} kind {spec.kind!r} (registered: {', '.join(sorted(table))})")
    return table[spec.kind](spec, dtype, device)
