"""Random-weights mode: a source of seeded tensors, and a writer of whole model folders.

The reference has no such mode in its public tree (its model tests read real files); this
one stands in for checkpoints everywhere here.  Matrices are N(0, std), biases N(0, bias_std),
norm weights 1 + N(0, norm_std).  The generator is counter-based: Philox4x32-10, the generator
of the reference's sampler (core/src/nn/sampling.cpp:207-227), keyed by (seed, hash of the
tensor's name) and counted by the element index, with a Box-Muller transform on top whose
logarithm, sine and cosine are short polynomials of individually rounded float32 operations.
So a tensor's values depend on nothing but the seed, its name and the position of each element,
and they are the same bits whether they are made here with numpy or on the GPU by the kernel
library's `sb_random_normal` (csrc/random_init.cu restates `normal_numpy` step for step): a
model made on the device equals the folder written from the same seed on a machine without one.
Values are rounded to bfloat16, the storage dtype of the folder.
"""
from __future__ import annotations

import json
import zlib
from pathlib import Path

import numpy as np
import torch

from .loader import TensorRequest
from .safetensors_io import write_safetensors

_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_STREAM = 0x5742          # third counter word: keeps these draws apart from the sampler's
_CHUNK = 1 << 20          # groups of four values made at a time


def tensor_key(seed: int, name: str) -> tuple:
    """The 64-bit Philox key of a tensor as two words."""
    seed = int(seed) & (2 ** 64 - 1)
    return seed & 0xffffffff, (zlib.crc32(name.encode("utf-8")) ^ (seed >> 32)) & 0xffffffff


def _philox(groups: np.ndarray, key0: int, key1: int) -> list:
    """Philox4x32-10 of counters {g_lo, g_hi, _STREAM, 0} for uint64 `groups`: four uint32 arrays."""
    mask = np.uint64(0xffffffff)
    c0, c1 = groups & mask, groups >> np.uint64(32)
    c2 = np.full_like(c0, _STREAM)
    c3 = np.zeros_like(c0)
    k0, k1 = key0, key1
    for _ in range(10):
        p0, p1 = np.uint64(_M0) * c0, np.uint64(_M1) * c2
        c0, c1, c2, c3 = ((p1 >> np.uint64(32)) ^ c1 ^ np.uint64(k0), p1 & mask,
                          (p0 >> np.uint64(32)) ^ c3 ^ np.uint64(k1), p0 & mask)
        k0, k1 = (k0 + _W0) & 0xffffffff, (k1 + _W1) & 0xffffffff
    return [c0, c1, c2, c3]


def _box_muller(wa: np.ndarray, wb: np.ndarray) -> tuple:
    """Two standard normal float32 arrays from two arrays of 32-bit words; every operation is
    one float32 operation, in the order csrc/random_init.cu performs them."""
    f32 = np.float32
    u1 = ((wa >> np.uint64(8)) + np.uint64(1)).astype(f32) * f32(2.0 ** -24)
    m, e = np.frexp(u1)
    low = m < f32(0.70710678)
    m = np.where(low, m * f32(2.0), m)
    e = np.where(low, e - 1, e)
    s = (m - f32(1.0)) / (m + f32(1.0))
    s2 = s * s
    p = f32(1.0 / 11.0)
    for c in (1.0 / 9.0, 1.0 / 7.0, 1.0 / 5.0, 1.0 / 3.0, 1.0):
        p = p * s2 + f32(c)
    ln_u1 = e.astype(f32) * f32(0.69314718) + (f32(2.0) * s) * p
    r = np.sqrt(f32(-2.0) * ln_u1)
    b = wb >> np.uint64(8)
    q, fb = b >> np.uint64(22), b & np.uint64(0x3fffff)
    fold = fb > np.uint64(0x200000)
    f = np.where(fold, np.uint64(0x400000) - fb, fb).astype(f32) * f32(2.0 ** -22)
    x = f * f32(1.57079633)
    x2 = x * x
    sp = f32(1.0 / 362880.0)
    for c in (-1.0 / 5040.0, 1.0 / 120.0, -1.0 / 6.0, 1.0):
        sp = sp * x2 + f32(c)
    sn = x * sp
    cp = f32(-1.0 / 3628800.0)
    for c in (1.0 / 40320.0, -1.0 / 720.0, 1.0 / 24.0, -1.0 / 2.0, 1.0):
        cp = cp * x2 + f32(c)
    cs = cp
    sn, cs = np.where(fold, cs, sn), np.where(fold, sn, cs)
    cos_t = np.select([q == 0, q == 1, q == 2], [cs, -sn, -cs], sn)
    sin_t = np.select([q == 0, q == 1, q == 2], [sn, cs, -sn], -cs)
    return r * cos_t, r * sin_t


def normal_numpy(n: int, key0: int, key1: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    """float32 [n]: mean + std * z with z standard normal, a function of the key and the element
    index only."""
    out = np.empty((n + 3) // 4 * 4, dtype=np.float32)
    mean, std = np.float32(mean), np.float32(std)
    for g0 in range(0, (n + 3) // 4, _CHUNK):
        groups = np.arange(g0, min(g0 + _CHUNK, (n + 3) // 4), dtype=np.uint64)
        w = _philox(groups, key0, key1)
        z = np.stack(_box_muller(w[0], w[1]) + _box_muller(w[2], w[3]), axis=1)   # [groups, 4]
        out[4 * g0:4 * g0 + z.size] = (mean + std * z).reshape(-1)
    return out[:n]


class RandomSource:
    """Looks like a tensor file to the binder, but makes each tensor when asked: with numpy on
    the CPU, with the kernel library on a CUDA device; the values are the same."""

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
        if r.role == "table":
            return torch.zeros(r.shape, dtype=torch.int32, device=self.device)
        mean, std = {"norm": (1.0, self.norm_std), "bias": (0.0, self.bias_std)}.get(
            r.role, (0.0, self.std))
        key0, key1 = tensor_key(self.seed, name)
        n = int(np.prod(r.shape, dtype=np.int64)) if len(r.shape) else 1
        if self.device.type == "cuda":
            from .. import ops
            with torch.cuda.device(self.device):
                out = torch.empty(r.shape, dtype=self.dtype, device=self.device)
                return ops.random_normal(out, key0, key1, mean, std)
        x = torch.from_numpy(normal_numpy(n, key0, key1, mean, std)).reshape(r.shape)
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
