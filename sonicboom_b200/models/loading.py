"""From a model folder (or a configuration and a seed) to a bound model on the device.

The steps are the reference's `boom_llm_model_load` (capi/src/capi.cpp:2066-2129) with its
file formats replaced: read config.json, pick the architecture from the registry, build the
model from its parts, ask the parts which tensors they want, check all of them against the
file at once, then bind."""
from __future__ import annotations

import torch

from ..config import read_config_json, spec_from_config_dict
from ..weights import RandomSource, SafetensorsDir, check, fetch
from .decoder import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")
    return _DTYPES[dtype]


def _bind(model: DecoderModel, source) -> DecoderModel:
    check(source, model.tensor_requests())
    model.bind(lambda name: fetch(source, name, model.dtype, model.device))
    return model


def load_model(model_dir, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """The model class is chosen by config.json's architectures[0], here as everywhere."""
    config_dict = read_config_json(model_dir)
    cfg, spec = spec_from_config_dict(config_dict)
    model = DecoderModel(spec, parse_dtype(dtype), device)
    model.config = cfg
    return _bind(model, SafetensorsDir(model_dir))


def random_model(config_dict: dict, seed: int, dtype="bfloat16", device="cuda:0", std=0.02,
                 bias_std=None, norm_std=0.0) -> DecoderModel:
    """A model with seeded random weights made directly on the device (no file)."""
    cfg, spec = spec_from_config_dict(config_dict)
    model = DecoderModel(spec, parse_dtype(dtype), device)
    model.config = cfg
    source = RandomSource(model.tensor_requests(), seed, std, bias_std, norm_std, device=device)
    return _bind(model, source)
