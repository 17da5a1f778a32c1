"""Binding weights by tensor name, with one error for everything that is wrong.

The model's parts say which tensors they need (`TensorRequest`); `check` compares that list
with what a source holds and raises once, listing missing tensors, unexpected tensors and
wrong shapes together, as the reference's binder accumulates every error before failing
(core/src/model/loader.cpp:325-408, 932).  `fetch` then brings one tensor to the device in
the dtype the engine keeps it in.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class TensorRequest:
    name: str
    shape: tuple
    role: str = "matrix"        # matrix | embedding | bias | norm | table (integers)
    optional: bool = False      # absent is fine, present is not "unexpected"


class WeightError(ValueError):
    """Raised once per load; the lists are also available as attributes."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_type=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_type = list(wrong_shape), list(wrong_type)
        lines = [f"weights do not match the model: {len(self.missing)} missing, "
                 f"{len(self.unexpected)} unexpected, {len(self.wrong_shape)} with a wrong shape, "
                 f"{len(self.wrong_type)} with a wrong type"]
        lines += [f"  missing tensor: {n} (expected shape {list(s)})" for n, s in self.missing]
        lines += [f"  unexpected tensor: {n} (shape {list(s)})" for n, s in self.unexpected]
        lines += [f"  tensor shape mismatch: {n} (expected {list(want)}, file has {list(got)})"
                  for n, want, got in self.wrong_shape]
        lines += [f"  tensor type mismatch: {n} ({why})" for n, why in self.wrong_type]
        super().__init__("\n".join(lines))


def check(source, requests) -> None:
    """Raises WeightError unless `source` holds exactly the requested tensors."""
    wanted = {}
    for r in requests:
        if r.name in wanted and tuple(wanted[r.name].shape) != tuple(r.shape):
            raise ValueError(f"two parts ask for {r.name} with different shapes")
        wanted.setdefault(r.name, r)
    have = set(source.names())
    missing, unexpected, wrong_shape, wrong_type = [], [], [], []
    for name, r in wanted.items():
        if name not in have:
            if not r.optional:
                missing.append((name, r.shape))
            continue
        dtype, shape = source.info(name)
        if tuple(shape) != tuple(r.shape):
            wrong_shape.append((name, r.shape, shape))
        if r.role == "table":
            if dtype.is_floating_point:
                wrong_type.append((name, f"integer table stored as {dtype}"))
        elif not dtype.is_floating_point:
            wrong_type.append((name, f"floating-point tensor stored as {dtype}"))
    for name in sorted(have - set(wanted)):
        if name.endswith("rotary_emb.inv_freq"):     # derived buffer some exporters store
            continue
        unexpected.append((name, source.info(name)[1]))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(missing, unexpected, wrong_shape, wrong_type)


def kept_dtype(stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """Dtype a stored tensor is kept in.  Serving (bfloat16): 16-bit floats are kept as
    bfloat16, a tensor stored in 32 bits stays so, integer tables are int32.  The float32
    path keeps every floating-point tensor in float32."""
    if not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def fetch(source, name: str, compute: torch.dtype, device) -> torch.Tensor:
    t = source.tensor(name)
    return t.to(device=device, dtype=kept_dtype(t.dtype, compute)).contiguous()
