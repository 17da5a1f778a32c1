"""Typed configurations, the model-as-parts records and the architecture registry."""
from .specs import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                    PositionSpec, ScheduleEntry)
from .registry import (ARCHITECTURES, Architecture, architecture_name, lookup, read_config_json,
                       register_architecture, spec_from_config_dict)
from .qwen2 import Qwen2Config

register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict, Qwen2Config.to_spec)

__all__ = ["ConfigError", "FeedForwardSpec", "LayerSpec", "MixerSpec", "ModelSpec", "NormSpec",
           "PositionSpec", "ScheduleEntry", "ARCHITECTURES", "Architecture", "architecture_name",
           "lookup", "read_config_json", "register_architecture", "spec_from_config_dict",
           "Qwen2Config"]
