"""Typed configuration of the Qwen2.5 dense decoder, read from its own config.json keys.

Counterpart of the reference's per-architecture metadata reader
(core/src/model/loader.cpp:628-685) and `Gemma4Config::valid`
(core/src/model/config.cpp:21-49): every size comes from the file, a missing or ill-typed
key is reported by name, and the constants that are fixed for this architecture
(score scale 1/sqrt(head_dim), q/k/v bias on, output and MLP bias off, half-split rotation of
the whole head, SiLU, pre-norm residual layout: core/src/model/recipe.cpp:65-70,153-160)
are written into the part records by `to_spec`, not into the parts.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

from .specs import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                    PositionSpec, ScheduleEntry)

_MISSING = object()


def _get(d: dict, key: str, kind, default=_MISSING, positive=False):
    """Reads one key with its type; errors name the key as the reference's
    "missing/invalid metadata: <key>" does (core/src/model/loader.cpp:641-654)."""
    v = d.get(key, None)
    if v is None:
        if default is _MISSING:
            raise ConfigError(f"missing/invalid config key: {key} (absent)")
        return default
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"missing/invalid config key: {key} (expected an integer, got {v!r})")
    elif kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"missing/invalid config key: {key} (expected a number, got {v!r})")
        v = float(v)
    elif kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"missing/invalid config key: {key} (expected true/false, got {v!r})")
    if positive and not v > 0:
        raise ConfigError(f"missing/invalid config key: {key} (must be > 0, got {v!r})")
    return v


@dataclass(frozen=True)
class Qwen2Config:
    """config.json of `Qwen2ForCausalLM`, typed."""
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    layer_types: tuple = ()
    eos_token_ids: tuple = ()
    architecture: str = "Qwen2ForCausalLM"

    @classmethod
    def from_dict(cls, d: dict) -> "Qwen2Config":
        hidden = _get(d, "hidden_size", int, positive=True)
        layers = _get(d, "num_hidden_layers", int, positive=True)
        heads = _get(d, "num_attention_heads", int, positive=True)
        kv_heads = _get(d, "num_key_value_heads", int, default=heads, positive=True)
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _get(d, "head_dim", int, positive=True)
        else:
            if hidden % heads:
                raise ConfigError("missing/invalid config key: head_dim (absent, and hidden_size "
                                  f"{hidden} is not a multiple of num_attention_heads {heads})")
            head_dim = hidden // heads          # core/src/model/loader.cpp:662
        inter = _get(d, "intermediate_size", int, positive=True)
        vocab = _get(d, "vocab_size", int, positive=True)
        max_pos = _get(d, "max_position_embeddings", int, positive=True)
        eps = _get(d, "rms_norm_eps", float, default=1e-6)
        if eps < 0:
            raise ConfigError("missing/invalid config key: rms_norm_eps (must be >= 0)")
        theta = _get(d, "rope_theta", float, default=10000.0, positive=True)
        tied = _get(d, "tie_word_embeddings", bool, default=False)
        use_window = _get(d, "use_sliding_window", bool, default=False)
        window = _get(d, "sliding_window", int, default=0)
        max_window_layers = _get(d, "max_window_layers", int, default=layers)
        layer_types = d.get("layer_types") or ()
        if d.get("rope_scaling") is not None:
            raise ConfigError("unsupported config key: rope_scaling (scaled rotary frequencies "
                              "are not built)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"unsupported config key: hidden_act = {act!r} (only 'silu')")
        if heads % kv_heads:
            raise ConfigError(f"missing/invalid config key: num_key_value_heads ({kv_heads} does not "
                              f"divide num_attention_heads {heads})")   # config.cpp:28
        if head_dim % 2:
            raise ConfigError(f"missing/invalid config key: head_dim ({head_dim} is odd; the "
                              "rotation pairs halves of a head)")        # nn/rope.cpp:61
        if use_window and window <= 0:
            raise ConfigError("missing/invalid config key: sliding_window (use_sliding_window is "
                              "true, so it must be > 0)")
        if layer_types:
            if len(layer_types) != layers:
                raise ConfigError(f"missing/invalid config key: layer_types (has {len(layer_types)} "
                                  f"entries for {layers} layers)")
            for t in layer_types:
                if t not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"unsupported config key: layer_types entry {t!r}")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError("missing/invalid config key: eos_token_id (an integer or a list)")
        return cls(hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                   num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
                   vocab_size=vocab, max_position_embeddings=max_pos, rms_norm_eps=eps,
                   rope_theta=theta, tie_word_embeddings=tied, use_sliding_window=use_window,
                   sliding_window=window if use_window else 0,
                   max_window_layers=max_window_layers, layer_types=tuple(layer_types),
                   eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        """config.json content that `from_dict` reads back to an equal configuration."""
        d = {
            "architectures": [self.architecture], "model_type": "qwen2",
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings, "hidden_act": "silu",
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window if self.use_sliding_window else None,
            "max_window_layers": self.max_window_layers, "torch_dtype": "bfloat16",
        }
        if self.layer_types:
            d["layer_types"] = list(self.layer_types)
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        return d

    def layer_window(self, i: int) -> int:
        """Window of layer i (0 = all keys).  With use_sliding_window, the layers from
        max_window_layers on are windowed unless layer_types names each layer's kind."""
        if not self.use_sliding_window:
            return 0
        if self.layer_types:
            return self.sliding_window if self.layer_types[i] == "sliding_attention" else 0
        return self.sliding_window if i >= self.max_window_layers else 0

    def to_spec(self) -> ModelSpec:
        """The model as parts: one pre-norm block per layer, run once each in order."""
        d, hd = self.hidden_size, self.head_dim
        scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))   # recipe.cpp:167
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            mixer = MixerSpec(
                kind="attention", width=d, n_heads=self.num_attention_heads,
                n_kv_heads=self.num_key_value_heads, head_dim=hd, window=self.layer_window(i),
                scale=scale, qkv_bias=True, out_bias=False,
                position=PositionSpec(kind="rope_neox", head_dim=hd, theta=self.rope_theta),
                prefix=p + "self_attn.")
            ffn = FeedForwardSpec(kind="swiglu", width=d, intermediate=self.intermediate_size,
                                  activation="silu", prefix=p + "mlp.")
            layers.append(LayerSpec(
                arrangement="pre_norm", mixer=mixer,
                mixer_norm=NormSpec("rmsnorm", d, self.rms_norm_eps, p + "input_layernorm.weight"),
                feed_forward=ffn,
                feed_forward_norm=NormSpec("rmsnorm", d, self.rms_norm_eps,
                                           p + "post_attention_layernorm.weight")))
        spec = ModelSpec(
            architecture=self.architecture, width=d, vocab=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding_tensor="model.embed_tokens.weight", layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=NormSpec("rmsnorm", d, self.rms_norm_eps, "model.norm.weight"),
            head_tensor=None if self.tie_word_embeddings else "lm_head.weight",
            stop_tokens=self.eos_token_ids)
        spec.validate()
        return spec
