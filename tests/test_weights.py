"""Safetensors reading and writing, binding errors, the random-weights mode (no device)."""
import json
import struct

import pytest
import torch

from conftest import TINY
from sonicboom_b200.config import spec_from_config_dict
from sonicboom_b200.models import tensor_requests
from sonicboom_b200.weights import (RandomSource, SafetensorsDir, SafetensorsError,
                                    SafetensorsFile, TensorRequest, WeightError, check, fetch,
                                    kept_dtype, write_random_model, write_safetensors)


def _file(tmp_path, header: dict, data: bytes, name="x.safetensors"):
    blob = json.dumps(header).encode()
    p = tmp_path / name
    p.write_bytes(struct.pack("<Q", len(blob)) + blob + data)
    return p


def test_round_trip(tmp_path):
    tensors = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32),
               "c": torch.randn(2, 2, 2), "d": torch.randn(4).half(), "e": torch.empty(0, 3)}
    write_safetensors(tmp_path / "t.safetensors", tensors, metadata={"k": "v"})
    f = SafetensorsFile(tmp_path / "t.safetensors")
    assert sorted(f.names()) == sorted(tensors)
    for n, t in tensors.items():
        assert f.info(n) == (t.dtype, tuple(t.shape))
        assert torch.equal(f.tensor(n), t)


def test_malformed_files(tmp_path):
    with pytest.raises(SafetensorsError, match="no such file"):
        SafetensorsFile(tmp_path / "none")
    (tmp_path / "short").write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(tmp_path / "short")
    (tmp_path / "trunc").write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="truncated header"):
        SafetensorsFile(tmp_path / "trunc")
    (tmp_path / "json").write_bytes(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="malformed header"):
        SafetensorsFile(tmp_path / "json")
    ok = {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}
    with pytest.raises(SafetensorsError, match="unknown dtype"):
        SafetensorsFile(_file(tmp_path, {"a": dict(ok, dtype="F99")}, b"\0" * 8))
    with pytest.raises(SafetensorsError, match="needs 8 bytes"):
        SafetensorsFile(_file(tmp_path, {"a": dict(ok, data_offsets=[0, 4])}, b"\0" * 8))
    with pytest.raises(SafetensorsError, match="outside the data section"):
        SafetensorsFile(_file(tmp_path, {"a": ok}, b"\0" * 4))
    with pytest.raises(SafetensorsError, match="overlap"):
        SafetensorsFile(_file(tmp_path, {"a": ok, "b": dict(ok, data_offsets=[4, 12])}, b"\0" * 12))
    with pytest.raises(SafetensorsError, match="malformed entry"):
        SafetensorsFile(_file(tmp_path, {"a": {"dtype": "F32"}}, b""))


def test_sharded_folder(tmp_path):
    write_safetensors(tmp_path / "s1.safetensors", {"a": torch.ones(2)})
    write_safetensors(tmp_path / "s2.safetensors", {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    d = SafetensorsDir(tmp_path)
    assert sorted(d.names()) == ["a", "b"] and d.tensor("b").shape == (3,)
    with pytest.raises(SafetensorsError, match="neither"):
        SafetensorsDir(tmp_path / "empty")


def test_one_error_lists_everything(tmp_path):
    _, spec = spec_from_config_dict(TINY["B"])
    requests = tensor_requests(spec)
    src = RandomSource(requests, seed=1)
    tensors = {n: src.tensor(n) for n in src.names()}
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.mlp.up_proj.weight"] = torch.zeros(512, 100).bfloat16()
    tensors["model.layers.9.extra.weight"] = torch.zeros(3).bfloat16()
    tensors["model.norm.weight"] = torch.zeros(192, dtype=torch.int32)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        check(SafetensorsDir(tmp_path), requests)
    err = e.value
    assert {n for n, _ in err.missing} == {"model.layers.1.self_attn.k_proj.bias", "lm_head.weight"}
    assert [n for n, _ in err.unexpected] == ["model.layers.9.extra.weight"]
    assert [(n, tuple(got)) for n, _, got in err.wrong_shape] == \
        [("model.layers.0.mlp.up_proj.weight", (512, 100))]
    assert [n for n, _ in err.wrong_type] == ["model.norm.weight"]
    text = str(err)
    for piece in ("missing tensor: lm_head.weight", "unexpected tensor: model.layers.9.extra.weight",
                  "shape mismatch: model.layers.0.mlp.up_proj.weight", "[512, 192]", "[512, 100]"):
        assert piece in text


def test_tied_model_may_carry_a_head(tmp_path):
    _, spec = spec_from_config_dict(TINY["A"])
    requests = tensor_requests(spec)
    assert "lm_head.weight" not in RandomSource(requests, 0).names()
    d = write_random_model(tmp_path / "m", TINY["A"], seed=3)
    check(SafetensorsDir(d), requests)
    tensors = {n: SafetensorsDir(d).tensor(n).clone() for n in SafetensorsDir(d).names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    write_safetensors(d / "model.safetensors", tensors)
    check(SafetensorsDir(d), requests)          # neither is "unexpected"


def test_random_mode_is_seeded_and_per_tensor(tmp_path):
    a = write_random_model(tmp_path / "a", TINY["A"], seed=5, std=0.02, norm_std=0.05)
    b = write_random_model(tmp_path / "b", TINY["A"], seed=5, std=0.02, norm_std=0.05)
    c = write_random_model(tmp_path / "c", TINY["A"], seed=6, std=0.02, norm_std=0.05)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    assert json.loads((a / "config.json").read_text()) == TINY["A"]
    f = SafetensorsDir(a)
    w = f.tensor("model.layers.0.mlp.up_proj.weight").float()
    n = f.tensor("model.norm.weight").float()
    assert f.info("model.norm.weight")[0] == torch.bfloat16
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(n.mean()) - 1.0) < 0.03
    # a tensor's values depend on (seed, name) only, not on the rest of the model
    _, spec = spec_from_config_dict(dict(TINY["A"], num_hidden_layers=1))
    one = RandomSource(tensor_requests(spec), 5, 0.02, None, 0.05)
    assert torch.equal(one.tensor("model.layers.0.mlp.up_proj.weight"),
                       f.tensor("model.layers.0.mlp.up_proj.weight"))


def test_kept_dtypes():
    bf, f32 = torch.bfloat16, torch.float32
    assert kept_dtype(bf, bf) == bf and kept_dtype(torch.float16, bf) == bf
    assert kept_dtype(f32, bf) == f32                    # stored in 32-bit: stays so
    assert kept_dtype(torch.int64, bf) == torch.int32 == kept_dtype(torch.int32, f32)
    assert kept_dtype(bf, f32) == f32 and kept_dtype(torch.float16, f32) == f32

    class Src:
        def tensor(self, name):
            return torch.ones(2, 2, dtype=torch.float16)
    assert fetch(Src(), "x", bf, "cpu").dtype == bf


# ------------------------------------------------------------------ the counter-based generator
def test_random_tensors_depend_on_seed_name_and_index_only():
    """Values are a function of (seed, tensor name, element index): the same prefix whatever the
    length, no dependence on how the work is cut, other values for another seed or name, and a
    normal distribution."""
    import numpy as np
    from sonicboom_b200.weights import random_init as ri
    k = ri.tensor_key(7, "model.layers.0.mlp.up_proj.weight")
    a = ri.normal_numpy(10_001, *k)
    assert a.dtype == np.float32 and a.shape == (10_001,)
    assert np.array_equal(ri.normal_numpy(37, *k), a[:37])
    old = ri._CHUNK
    try:
        ri._CHUNK = 64                            # chunks of 256 values
        assert np.array_equal(ri.normal_numpy(10_001, *k), a)
    finally:
        ri._CHUNK = old
    assert not np.array_equal(ri.normal_numpy(64, *ri.tensor_key(8, "model.layers.0.mlp.up_proj.weight")), a[:64])
    assert not np.array_equal(ri.normal_numpy(64, *ri.tensor_key(7, "model.layers.1.mlp.up_proj.weight")), a[:64])
    assert ri.tensor_key(7 + 2 ** 32, "x") != ri.tensor_key(7, "x")      # the upper seed bits count
    z = ri.normal_numpy(400_000, *k).astype(np.float64)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01
    assert abs((z ** 3).mean()) < 0.03 and abs((z ** 4).mean() - 3.0) < 0.1
    assert 4.0 < np.abs(z).max() < 7.0
    # the words are Philox4x32-10 of {group, 0x5742, 0} under the tensor's key
    import plain_sampling as ps
    w = ri._philox(np.asarray([5, 2 ** 33 + 1], dtype=np.uint64), *k)
    assert [int(x[0]) for x in w] == ps.philox4x32_10((5, 0, 0x5742, 0), k[0] | (k[1] << 32))
    assert [int(x[1]) for x in w] == ps.philox4x32_10((1, 2, 0x5742, 0), k[0] | (k[1] << 32))
    shifted = ri.normal_numpy(8, *k, mean=1.0, std=0.05)
    assert np.array_equal(shifted, np.float32(1.0) + np.float32(0.05) * a[:8])


def test_random_source_roles_and_folder(tmp_path):
    cfg = dict(architectures=["Qwen2ForCausalLM"], hidden_size=32, num_hidden_layers=1,
               num_attention_heads=2, num_key_value_heads=1, intermediate_size=48, vocab_size=50,
               max_position_embeddings=64, tie_word_embeddings=True)
    write_random_model(tmp_path, cfg, seed=3, std=0.5, bias_std=0.25, norm_std=0.125)
    st = SafetensorsDir(tmp_path)
    from sonicboom_b200.weights import random_init as ri
    for name, mean, std in [("model.layers.0.self_attn.q_proj.weight", 0.0, 0.5),
                            ("model.layers.0.self_attn.k_proj.bias", 0.0, 0.25),
                            ("model.norm.weight", 1.0, 0.125)]:
        t = st.tensor(name)
        want = torch.from_numpy(ri.normal_numpy(t.numel(), *ri.tensor_key(3, name), mean, std))
        assert torch.equal(t.float().reshape(-1), want.to(torch.bfloat16).float())
