"""The plain implementation against the reference's own compiled CPU primitives.

tests/golden/reference_primitives.json was written by tests/golden/make_golden.py, which compiles
hardenedlinux/SonicBoom's core/src/nn/*.cpp in place and runs them in the emitter's order for one
Qwen2 block, the head and the sampler.  This test needs only the committed JSON."""
import json
import sys
from pathlib import Path

import numpy as np
import torch

import plain_model as pm
import plain_sampling as ps

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN_DIR))
from make_golden import CFG, make_inputs  # noqa: E402


def _load():
    g = json.loads((GOLDEN_DIR / "reference_primitives.json").read_text())
    assert g["config"] == CFG
    t = {k: torch.from_numpy(v) for k, v in make_inputs().items()}
    return g, t


def close(got, want, shape, tol=2e-6):
    want = torch.tensor(want, dtype=torch.float32).reshape(shape)
    err = pm.rel_err(got.reshape(shape), want)
    assert err < tol, err


def test_block_parts_match_the_reference_primitives():
    g, t = _load()
    c = CFG
    n, d, hq, hkv, hd, ff = c["n"], c["d"], c["hq"], c["hkv"], c["hd"], c["ff"]
    pos = torch.arange(n)
    h = pm.rms_norm(t["x"], t["wn1"], c["eps"])
    close(h, g["normed"], (n, d))
    q = pm.rope_neox(pm.linear(h, t["wq"], t["bq"]).view(n, hq, hd), pos, c["theta"])
    k = pm.rope_neox(pm.linear(h, t["wk"], t["bk"]).view(n, hkv, hd), pos, c["theta"])
    v = pm.linear(h, t["wv"], t["bv"]).view(n, hkv, hd)
    close(q, g["q_rotated"], (n, hq, hd))
    close(k, g["k_rotated"], (n, hkv, hd))
    close(v, g["v"], (n, hkv, hd))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    att = pm.attention(q, k, v, pos, pos, scale)
    close(att, g["attention"], (n, hq, hd))
    close(pm.attention(q, k, v, pos, pos, scale, window=c["window"]), g["attention_window"], (n, hq, hd))
    close(att[-1], g["decode_attention"], (hq, hd))           # decode = the last row of prefill
    x1 = pm.linear(att.reshape(n, hq * hd), t["wo"]) + t["x"]
    f = pm.rms_norm(x1, t["wn2"], c["eps"])
    act = pm.silu(pm.linear(f, t["wgate"])) * pm.linear(f, t["wup"])
    close(act, g["swiglu_act"], (n, ff))
    x2 = pm.linear(act, t["wdown"]) + x1
    close(x2, g["block_out"], (n, d))
    logits = pm.linear(pm.rms_norm(x2, t["wnf"], c["eps"]), t["whead"])
    close(logits, g["logits"], (n, c["vocab"]))


def test_whole_model_function_matches_too():
    """The same through plain_model.forward: a one-layer model folder's worth of tensors."""
    g, t = _load()
    c = CFG
    cfg = dict(num_hidden_layers=1, hidden_size=c["d"], num_attention_heads=c["hq"],
               num_key_value_heads=c["hkv"], head_dim=c["hd"], rms_norm_eps=c["eps"], rope_theta=c["theta"],
               tie_word_embeddings=False)
    p = "model.layers.0."
    tensors = {"model.embed_tokens.weight": t["x"], p + "input_layernorm.weight": t["wn1"],
               p + "self_attn.q_proj.weight": t["wq"], p + "self_attn.q_proj.bias": t["bq"],
               p + "self_attn.k_proj.weight": t["wk"], p + "self_attn.k_proj.bias": t["bk"],
               p + "self_attn.v_proj.weight": t["wv"], p + "self_attn.v_proj.bias": t["bv"],
               p + "self_attn.o_proj.weight": t["wo"], p + "post_attention_layernorm.weight": t["wn2"],
               p + "mlp.up_proj.weight": t["wup"], p + "mlp.gate_proj.weight": t["wgate"],
               p + "mlp.down_proj.weight": t["wdown"], "model.norm.weight": t["wnf"], "lm_head.weight": t["whead"]}
    logits = pm.forward(cfg, tensors, list(range(c["n"])))     # token i embeds to row i of x
    close(logits, g["logits"], (c["n"], c["vocab"]))


def test_sampler_and_philox_match_the_reference():
    g, _ = _load()
    c = CFG
    logits = np.asarray(g["logits"], dtype=np.float32).reshape(c["n"], c["vocab"])[-1]
    want = [int(x) for x in g["sample_tokens"]]
    history = [3, 7, 7, 11, 3, 7]
    got = [ps.argmax(logits)]
    cases = [(0.0, 0, 1.0, 0.0, 0, 1.0, 0, 0, 64), (0.8, 0, 1.0, 0.0, 5, 1.0, 0, 0, 64),
             (1.5, 5, 1.0, 0.0, 1, 1.0, 0, 0, 64), (1.0, 0, 0.6, 0.0, 9, 1.0, 0, 0, 64),
             (0.7, 0, 1.0, 0.2, 3, 1.0, 0, 0, 64), (0.9, 0, 1.0, 0.0, 4, 1.3, 0.5, 0.25, 4),
             (0.0, 0, 1.0, 0.0, 0, 5.0, 9.0, 0, 64), (2.0, 20, 0.9, 0.01, 1 << 40, 1.1, 0.1, 0.1, 3)]
    for t_, k, p, minp, seed, rp, pp, fp, last_n in cases:
        for pos in (0, 17, (1 << 33) + 1):
            params = ps.Params(t_, k, p, minp, seed, rp, last_n, pp, fp)
            got.append(ps.sample_token(logits, params, pos, history))
    assert got == want
    ph = ps.philox4x32_10([1, 2, 3, 4], 0x123456789abcdef)
    assert [ph[0] >> 16, ph[0] & 0xffff, ph[1] >> 16, ph[1] & 0xffff] == [int(x) for x in g["philox"]]
