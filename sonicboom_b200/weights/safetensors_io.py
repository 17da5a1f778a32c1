"""Reading and writing .safetensors files without any library for the format.

Layout (as the reference's own reader parses it, core/src/safetensors/reader.cpp:178-367):
an 8-byte little-endian header length, a JSON directory {name: {dtype, shape, data_offsets}}
and the data section; offsets are relative to the data section.  The same malformed-file
checks are made: truncated header, malformed JSON, unknown dtype, shape x dtype size
different from the offsets' span, a range past the data section, overlapping ranges.
A folder may hold one `model.safetensors` or shards named by
`model.safetensors.index.json`'s `weight_map` (reader.cpp:395-448).
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path

import torch

DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped file; tensors are handed out as CPU views of the mapping."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise SafetensorsError(f"{self.path}: no such file")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: truncated (no header length)")
        self._fh = open(self.path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: truncated header ({hlen} bytes announced, "
                                   f"{size - 8} present)")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: malformed header JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header is not an object")
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: dict[str, tuple] = {}
        spans = []
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype_name, shape, (b, e) = info["dtype"], info["shape"], info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: malformed entry for {name!r}") from None
            if dtype_name not in DTYPES:
                raise SafetensorsError(f"{self.path}: {name}: unknown dtype {dtype_name!r}")
            dtype, width = DTYPES[dtype_name]
            count = 1
            for s in shape:
                if not isinstance(s, int) or s < 0:
                    raise SafetensorsError(f"{self.path}: {name}: bad shape {shape}")
                count *= s
            if e - b != count * width:
                raise SafetensorsError(f"{self.path}: {name}: shape {shape} of {dtype_name} needs "
                                       f"{count * width} bytes, offsets span {e - b}")
            if b < 0 or e > data_len:
                raise SafetensorsError(f"{self.path}: {name}: range [{b}, {e}) is outside the data "
                                       f"section of {data_len} bytes")
            self.entries[name] = (dtype, tuple(shape), b, e)
            if e > b:
                spans.append((b, e, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{self.path}: ranges of {n0} and {n1} overlap")

    def names(self):
        return list(self.entries)

    def info(self, name):
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name) -> torch.Tensor:
        dtype, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._map)[self._data_start + b:self._data_start + e]
        with warnings.catch_warnings():      # the mapping is read-only; tensors of it are only read
            warnings.simplefilter("ignore", UserWarning)
            return torch.frombuffer(view, dtype=dtype).reshape(shape)


class SafetensorsDir:
    """All tensors of a model folder: one file, or the shards its index names."""

    def __init__(self, model_dir):
        model_dir = Path(model_dir)
        index = model_dir / "model.safetensors.index.json"
        single = model_dir / "model.safetensors"
        self._where: dict[str, SafetensorsFile] = {}
        if single.is_file():
            files = [SafetensorsFile(single)]
        elif index.is_file():
            try:
                weight_map = json.loads(index.read_text())["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise SafetensorsError(f"{index}: no readable weight_map") from None
            files = [SafetensorsFile(model_dir / f) for f in sorted(set(weight_map.values()))]
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor "
                                   "model.safetensors.index.json")
        for f in files:
            for n in f.names():
                self._where[n] = f

    def names(self):
        return list(self._where)

    def info(self, name):
        return self._where[name].info(name)

    def tensor(self, name):
        return self._where[name].tensor(name)


def write_safetensors(path, tensors, metadata=None) -> None:
    """Writes {name: CPU tensor} (or an iterable of (name, dtype, shape, producer)) in name
    order.  A producer is called when its bytes are due, so a large model is never held whole."""
    items = []
    if isinstance(tensors, dict):
        for name, t in tensors.items():
            items.append((name, t.dtype, tuple(t.shape), (lambda t=t: t)))
    else:
        items = list(tensors)
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, dtype, shape, _ in items:
        if dtype not in _NAMES:
            raise SafetensorsError(f"{name}: dtype {dtype} cannot be stored")
        count = 1
        for s in shape:
            count *= s
        nbytes = count * DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-(8 + len(blob)) % 64)          # data section starts 64-byte aligned
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name, dtype, shape, produce in items:
            t = produce().detach().to("cpu").contiguous()
            if t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(f"{name}: produced {t.dtype} {tuple(t.shape)}, "
                                       f"announced {dtype} {tuple(shape)}")
            fh.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
