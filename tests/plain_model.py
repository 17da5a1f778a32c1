"""Plain, slow implementation of the Qwen2.5 dense decoder, used only as the test oracle.

Whole sequences, no cache, one function for each part, CPU torch in float32 (or
float64 on request).  It shares no code with the package under test: it has its
own safetensors reader, its own configuration reading and its own formulas.

Every function is written from the formulas of hardenedlinux/SonicBoom's CPU
primitives and model emitter and cites them (paths relative to that project).
The reference's model code needs its MLIR compiler and GGUF models and cannot be
built without them, so the whole-model arrangement here rests on the formulas of
core/src/model/emit.cpp; the primitives are checked once against the reference's
own compiled CPU primitives by tests/golden/make_golden.py.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# --------------------------------------------------------------------------- files


_ST_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2),
              "I32": (np.int32, 4), "I64": (np.int64, 8), "F64": (np.float64, 8)}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Reads every tensor of a .safetensors file as float32 (integers as int64).

    Format (core/src/safetensors/reader.cpp:178-367): 8-byte little-endian header
    length, a JSON directory {name: {dtype, shape, data_offsets}}, then the data
    section; offsets are relative to the data section.
    """
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    data = raw[8 + hlen:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        np_dtype, _ = _ST_DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        arr = np.frombuffer(data[b:e], dtype=np_dtype).reshape(info["shape"])
        if info["dtype"] == "BF16":
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        t = torch.from_numpy(np.array(arr))
        out[name] = t.to(torch.int64) if info["dtype"] in ("I32", "I64") else t.to(torch.float32)
    return out


def read_model_dir(model_dir):
    """Returns (config dict, {tensor name: float32 tensor}) of a model folder."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    return cfg, read_safetensors(model_dir / "model.safetensors")


# --------------------------------------------------------------------------- parts


def embedding(table: torch.Tensor, tokens) -> torch.Tensor:
    """x = E[token]; no sqrt(d) scale for Qwen2 (core/src/model/emit.cpp:237-247,
    core/src/nn/embedding.cpp:23-28)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """inv = 1/sqrt(mean(x^2)+eps); y = (x*inv)*w, plain weight (not 1+w); the mean
    is accumulated wider than float32 (core/src/nn/norm.cpp:25-42,
    core/src/nn/cpu_reduce.h:38-57)."""
    mean_sq = (x.to(torch.float64) ** 2).mean(dim=-1, keepdim=True).to(x.dtype)
    inv = 1.0 / torch.sqrt(mean_sq + eps)
    return x * inv * weight.to(x.dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y[j] = sum_i W[j][i] x[i], then y += b as a separate step
    (core/src/nn/matmul.cpp:26-38, core/src/nn/elementwise.cpp:52-59)."""
    y = x @ weight.to(x.dtype).t()
    if bias is not None:
        y = y + bias.to(x.dtype)
    return y


def rope_neox(x: torch.Tensor, positions: torch.Tensor, theta_base: float) -> torch.Tensor:
    """Half-split (NEOX) rotation of whole heads.  x: [n, heads, hd].  For i < hd/2:
    theta = pos * exp(-2i/hd * ln(base)) in float32, x'_i = x_i c - x_{i+hd/2} s,
    x'_{i+hd/2} = x_i s + x_{i+hd/2} c (core/src/nn/rope.cpp:26-55, 58-82)."""
    n, heads, hd = x.shape
    half = hd // 2
    i = torch.arange(half, dtype=torch.float32)
    log_base = torch.log(torch.tensor(theta_base, dtype=torch.float32))
    inv_freq = torch.exp(-2.0 * i / float(hd) * log_base)          # float32, as the reference
    theta = positions.to(torch.float32)[:, None] * inv_freq[None, :]  # [n, half]
    c = torch.cos(theta).to(x.dtype)[:, None, :]
    s = torch.sin(theta).to(x.dtype)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_positions: torch.Tensor,
              k_positions: torch.Tensor, scale: float, window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention, one query and one head at a time.

    q: [nq, Hq, hd]; k, v: [nk, Hkv, hd].  kv head = h // (Hq/Hkv); score = (q.k)*scale
    with the scale applied after the whole dot; key j is masked when j > i or (window > 0
    and i >= j + window); softmax with max subtraction; out = sum(e_j v_j)/sum(e_j)
    (core/src/nn/attention.cpp:26-105)."""
    nq, hq, hd = q.shape
    nk, hkv, _ = k.shape
    group = hq // hkv
    out = torch.zeros_like(q)
    for h in range(hq):
        kh = h // group
        scores = (q[:, h, :] @ k[:, kh, :].t()) * scale              # [nq, nk]
        i = q_positions[:, None]
        j = k_positions[None, :]
        masked = j > i
        if window > 0:
            masked = masked | (i >= j + window)
        scores = scores.masked_fill(masked, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        e = torch.where(masked, torch.zeros_like(e), e)
        out[:, h, :] = (e @ v[:, kh, :]) / e.sum(dim=-1, keepdim=True)
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x)) (core/src/nn/activation.cpp:41-50)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(x, w_gate, w_up, w_down) -> torch.Tensor:
    """u = Wup f; g = silu(Wgate f); y = Wdown (g*u); no biases
    (core/src/model/emit.cpp:364-374)."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


# --------------------------------------------------------------------------- model


def layer_windows(cfg: dict) -> list[int]:
    """Window (0 = all keys) of every layer from config.json: with use_sliding_window the
    layers from max_window_layers on see only the last sliding_window keys; a
    `layer_types` list, when present, names each layer's kind itself."""
    n = cfg["num_hidden_layers"]
    if not cfg.get("use_sliding_window", False) or not cfg.get("sliding_window"):
        return [0] * n
    w = int(cfg["sliding_window"])
    types = cfg.get("layer_types")
    if types:
        return [w if t == "sliding_attention" else 0 for t in types]
    first = cfg.get("max_window_layers", n)
    return [w if i >= first else 0 for i in range(n)]


def self_attention(h, positions, p, cfg, window, tensors, shared_kv=None):
    """Mixer of one block in emitter order: q matmul + bias, rope(q); k, v matmuls, then
    their biases, rope(k); attend; output projection without bias
    (core/src/model/emit.cpp:255-308).  K and V stay unrounded here.  Returns (out, (k, v));
    with `shared_kv` the block reads those keys and values and projects only queries."""
    hq = cfg["num_attention_heads"]
    hkv = cfg.get("num_key_value_heads", hq)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // hq
    n = h.shape[0]
    q = linear(h, tensors[p + "self_attn.q_proj.weight"], tensors.get(p + "self_attn.q_proj.bias"))
    q = rope_neox(q.view(n, hq, hd), positions, float(cfg.get("rope_theta", 10000.0)))
    if shared_kv is None:
        k = linear(h, tensors[p + "self_attn.k_proj.weight"], tensors.get(p + "self_attn.k_proj.bias"))
        v = linear(h, tensors[p + "self_attn.v_proj.weight"], tensors.get(p + "self_attn.v_proj.bias"))
        k = rope_neox(k.view(n, hkv, hd), positions, float(cfg.get("rope_theta", 10000.0)))
        v = v.view(n, hkv, hd)
    else:
        k, v = shared_kv
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))          # core/src/model/recipe.cpp:167
    a = attention(q, k, v, positions, positions, scale, window)
    return linear(a.reshape(n, hq * hd), tensors[p + "self_attn.o_proj.weight"]), (k, v)


def block(x, positions, layer, cfg, window, tensors, shared_kv=None):
    """Pre-norm residual block: h = norm(x); x1 = mix(h) + x; f = norm(x1); x2 = ffn(f) + x1
    (core/src/model/emit.cpp:436-459; no post norms, gate or output scale for Qwen2)."""
    p = f"model.layers.{layer}."
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    h = rms_norm(x, tensors[p + "input_layernorm.weight"], eps)
    mixed, kv = self_attention(h, positions, p, cfg, window, tensors, shared_kv)
    x1 = mixed + x
    f = rms_norm(x1, tensors[p + "post_attention_layernorm.weight"], eps)
    fed = swiglu_mlp(f, tensors[p + "mlp.gate_proj.weight"], tensors[p + "mlp.up_proj.weight"],
                     tensors[p + "mlp.down_proj.weight"])
    return fed + x1, kv


def forward(cfg: dict, tensors: dict, tokens, dtype=torch.float32, schedule=None) -> torch.Tensor:
    """Logits [n, vocab] at every position of one whole sequence.

    Embedding, the blocks in schedule order, final norm, LM head; a tied head uses the
    embedding matrix (core/src/model/emit.cpp:512-523, core/src/model/exec.cpp:516-517).
    `schedule` is a list of (layer index, index of the schedule entry whose keys and values
    are read, or None for its own); the default runs every layer once in order."""
    tensors = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    n = len(tokens)
    positions = torch.arange(n)
    x = embedding(tensors["model.embed_tokens.weight"], tokens)
    windows = layer_windows(cfg)
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    kvs = []
    for layer, source in schedule:
        shared = kvs[source] if source is not None else None
        x, kv = block(x, positions, layer, cfg, windows[layer], tensors, shared)
        kvs.append(kv)
    hn = rms_norm(x, tensors["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-6)))
    head = tensors["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else tensors["lm_head.weight"]
    return linear(hn, head)


def greedy_generate(cfg, tensors, prompt, max_tokens, stop_tokens=()) -> list[int]:
    """Greedy continuation by whole-sequence forwards: the argmax of the last position,
    ties toward the lowest id (core/src/nn/sampling.cpp:238-244); a stop token is
    emitted and ends the sequence (core/include/sonicboom/model/plan.h:438-440)."""
    seq = list(prompt)
    out = []
    for _ in range(max_tokens):
        logits = forward(cfg, tensors, seq)[-1]
        tok = int(torch.argmax(logits))      # torch.argmax returns the first maximum
        out.append(tok)
        seq.append(tok)
        if tok in stop_tokens:
            break
    return out


# --------------------------------------------------------------------------- comparing


def rel_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """Largest absolute difference relative to the reference's largest magnitude."""
    a = a.double()
    ref = ref.double()
    return float((a - ref).abs().max() / max(float(ref.abs().max()), 1e-12))


def sqrt_f32(x: float) -> float:
    return float(math.sqrt(np.float32(x)))
