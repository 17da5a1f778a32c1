"""Model description as data: what each layer is made of and in which order layers run.

A `ModelSpec` plays the role of the reference's `Recipe`
(core/include/sonicboom/model/recipe.h:51-205): parts carry their sizes and constants as
parameters, every layer names its own mixer and feed-forward, and the run order is a list
that may name a layer twice or let an entry read another entry's cache
(`SelfAttention.cache/owns_cache`, recipe.h:89-93).  Nothing here knows an architecture;
an architecture's configuration class fills these records in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


class ConfigError(ValueError):
    """A configuration that cannot be built; the message names the offending key."""


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer."""
    kind: str                      # key of parts.POSITION_ENCODINGS, e.g. "rope_neox"
    head_dim: int
    theta: float = 10000.0
    rotary_dim: int = 0            # 0 = the whole head is rotated


@dataclass(frozen=True)
class NormSpec:
    kind: str                      # key of parts.NORMS, e.g. "rmsnorm"
    width: int
    eps: float
    tensor: str                    # tensor name of the weight


@dataclass(frozen=True)
class MixerSpec:
    """Token mixer of one layer.  `params` holds what only that kind of mixer needs."""
    kind: str                      # key of parts.MIXERS, e.g. "attention"
    width: int                     # residual width in and out
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    window: int = 0                # 0 = every earlier key; n = the last n keys
    scale: float = 0.0             # score multiplier, applied after the dot product
    qkv_bias: bool = False
    out_bias: bool = False
    position: Optional[PositionSpec] = None
    prefix: str = ""               # tensor-name prefix, e.g. "model.layers.3.self_attn."
    params: tuple = ()             # extra (key, value) pairs for other mixer kinds


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                      # key of parts.FEED_FORWARDS, e.g. "swiglu"
    width: int
    intermediate: int
    activation: str = "silu"
    prefix: str = ""
    params: tuple = ()


@dataclass(frozen=True)
class LayerSpec:
    """One block: which arrangement, and the parts it arranges."""
    arrangement: str               # key of parts.BLOCKS, e.g. "pre_norm"
    mixer: MixerSpec
    mixer_norm: NormSpec
    feed_forward: FeedForwardSpec
    feed_forward_norm: NormSpec

    @property
    def kind(self) -> str:
        return self.arrangement


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `cache_from` is the index of an earlier schedule entry whose
    cache this run reads instead of writing its own (None: it owns a cache)."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    width: int
    vocab: int
    max_positions: int
    embedding_tensor: str
    layers: tuple                  # of LayerSpec
    schedule: tuple                # of ScheduleEntry
    final_norm: NormSpec = None
    head_tensor: Optional[str] = None   # None: the head is the embedding matrix (tied)
    stop_tokens: tuple = ()
    embedding_scale: float = 1.0        # multiplies every embedding row (1: as stored)
    logit_cap: float = 0.0              # c > 0: logits = c * tanh(logits / c); 0: no cap

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("model has no layers")
        if not self.embedding_scale > 0.0:
            raise ConfigError(f"embedding_scale {self.embedding_scale} must be positive")
        if self.logit_cap < 0.0:
            raise ConfigError(f"logit_cap {self.logit_cap} must be zero (none) or positive")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule[{i}] names layer {e.layer}, model has {len(self.layers)}")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ConfigError(f"schedule[{i}] reads the cache of entry {e.cache_from}, "
                                      "which does not run before it")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ConfigError(f"schedule[{i}] reads the cache of entry {e.cache_from}, "
                                      "which owns none")
