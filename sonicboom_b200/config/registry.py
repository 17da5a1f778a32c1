"""The one registry from an architecture's name to its configuration and model.

Counterpart of `detect_arch` / `load_config` (core/src/model/loader.cpp:847-865): the name
in config.json's `architectures[0]` selects everything; an unknown name is an
"unsupported" error that repeats the name (capi/src/capi.cpp:2090-2094).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from .specs import ConfigError, ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict], object]       # config.json dict -> typed configuration
    build_spec: Callable[[object], ModelSpec]    # typed configuration -> model as parts


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec) -> None:
    ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)


def architecture_name(config_dict: dict) -> str:
    archs = config_dict.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("missing/invalid config key: architectures (a non-empty list of names)")
    return archs[0]


def lookup(config_dict: dict) -> Architecture:
    name = architecture_name(config_dict)
    if name not in ARCHITECTURES:
        raise ConfigError(f"unsupported architecture: {name!r} (registered: "
                          f"{', '.join(sorted(ARCHITECTURES)) or 'none'})")
    return ARCHITECTURES[name]


def read_config_json(model_dir) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {model_dir}")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"config.json is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError("config.json does not hold an object")
    return d


def spec_from_config_dict(config_dict: dict):
    """(typed configuration, ModelSpec) for a config.json dictionary."""
    arch = lookup(config_dict)
    cfg = arch.parse_config(config_dict)
    return cfg, arch.build_spec(cfg)
