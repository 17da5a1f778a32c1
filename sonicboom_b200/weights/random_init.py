"""Random-weights mode: a source of seeded tensors, and a writer of whole model folders.

The reference has no such mode in its public tree (its model tests read real files); this
one stands in for checkpoints everywhere here.  Matrices are N(0, std), biases N(0, bias_std),
norm weights 1 + N(0, norm_std); every tensor's stream depends only on (seed, tensor name), so
a tensor's values do not depend on which other tensors exist.  Values are rounded to bfloat16,
the storage dtype of the folder.
"""
from __future__ import annotations

import json
import zlib
from pathlib import Path

import torch

from .loader import TensorRequest
from .safetensors_io import write_safetensors


class RandomSource:
    """Looks like a tensor file to the binder, but makes each tensor when asked."""

    def __init__(self, requests, seed: int, std=0.02, bias_std=None, norm_std=0.0,
                 dtype=torch.bfloat16, device="cpu"):
        self.requests = {r.name: r for r in requests if not r.optional}
        self.seed, self.std = int(seed), float(std)
        self.bias_std = float(std if bias_std is None else bias_std)
        self.norm_std = float(norm_std)
        self.dtype, self.device = dtype, torch.device(device)

    def names(self):
        return list(self.requests)

    def info(self, name):
        r = self.requests[name]
        return (torch.int32 if r.role == "table" else self.dtype), tuple(r.shape)

    def tensor(self, name) -> torch.Tensor:
        r = self.requests[name]
        gen = torch.Generator(device=self.device)
        gen.manual_seed((self.seed * 1000003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63))
        if r.role == "table":
            return torch.zeros(r.shape, dtype=torch.int32, device=self.device)
        x = torch.randn(r.shape, generator=gen, device=self.device, dtype=torch.float32)
        if r.role == "norm":
            x = 1.0 + self.norm_std * x
        elif r.role == "bias":
            x = self.bias_std * x
        else:
            x = self.std * x
        return x.to(self.dtype)


def write_random_model(model_dir, config_dict: dict, seed: int, std=0.02, bias_std=None,
                       norm_std=0.0, dtype=torch.bfloat16) -> Path:
    """Writes config.json and model.safetensors for `config_dict` with seeded random weights."""
    from ..config import spec_from_config_dict
    from ..models import tensor_requests

    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    _, spec = spec_from_config_dict(config_dict)
    src = RandomSource(tensor_requests(spec), seed, std, bias_std, norm_std, dtype)
    (model_dir / "config.json").write_text(json.dumps(config_dict, indent=1))
    items = [(n, src.info(n)[0], src.info(n)[1], (lambda n=n: src.tensor(n))) for n in src.names()]
    write_safetensors(model_dir / "model.safetensors", items,
                      metadata={"format": "pt", "seed": seed})
    return model_dir
