"""The plain implementation checked on its own: known values and invariants, the cases the
reference's primitive tests use (tests/core/test_nn.cpp:172-291, 402-470;
tests/core/test_sampling.cpp:42-117)."""
import math

import numpy as np
import torch

import plain_model as pm
import plain_sampling as ps
from conftest import TINY, prompts_for


def test_rms_norm_known_value_and_invariants():
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    y = pm.rms_norm(x, torch.ones(4), 0.0)
    assert abs(float(y[0, 0]) - 0.365148) < 1e-6          # 1/sqrt(7.5)
    assert torch.allclose(pm.rms_norm(3 * x, torch.ones(4), 0.0), y, atol=1e-6)   # scale invariant
    w = torch.tensor([2.0, 0.5, 1.0, 0.0])
    assert torch.allclose(pm.rms_norm(x, w, 0.0), y * w)
    assert float(pm.rms_norm(torch.zeros(1, 4), torch.ones(4), 1e-6).abs().max()) == 0.0
    big_eps = pm.rms_norm(x, torch.ones(4), 100.0)
    assert torch.allclose(big_eps, x / math.sqrt(107.5), atol=1e-6)


def test_rope_identity_quarter_turn_and_norm():
    x = torch.randn(1, 3, 8)
    assert torch.equal(pm.rope_neox(x, torch.tensor([0]), 10000.0), x)        # position 0
    # pair 0 has frequency 1: position pi/2 turns (1, 0) into (0, 1); pairs are (i, i + hd/2)
    v = torch.zeros(1, 1, 4); v[0, 0, 0] = 1.0
    inv = math.exp(-2.0 * 0 / 4 * math.log(10000.0))
    pos = torch.tensor([1])
    r = pm.rope_neox(v, pos, 10000.0)
    assert abs(float(r[0, 0, 0]) - math.cos(1.0)) < 1e-6 and abs(float(r[0, 0, 2]) - math.sin(1.0)) < 1e-6
    assert float(r[0, 0, 1]) == 0.0 and float(r[0, 0, 3]) == 0.0
    y = pm.rope_neox(x.repeat(5, 1, 1), torch.arange(5) * 1000, 1e6)
    assert torch.allclose(y.norm(dim=-1), x.repeat(5, 1, 1).norm(dim=-1), atol=1e-5)
    # relative property: q(m).k(n) depends on m - n only
    q, k = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    d1 = (pm.rope_neox(q, torch.tensor([7]), 1e4) * pm.rope_neox(k, torch.tensor([3]), 1e4)).sum()
    d2 = (pm.rope_neox(q, torch.tensor([104]), 1e4) * pm.rope_neox(k, torch.tensor([100]), 1e4)).sum()
    assert abs(float(d1 - d2)) < 1e-4


def test_attention_single_key_causal_groups_window():
    hd = 4
    q = torch.randn(1, 2, hd)
    k, v = torch.randn(1, 1, hd), torch.randn(1, 1, hd)
    out = pm.attention(q, k, v, torch.tensor([0]), torch.tensor([0]), 0.5)
    assert torch.allclose(out, v.expand(1, 2, hd))                            # one key: out = v
    n = 6
    q, k, v = torch.randn(n, 4, hd), torch.randn(n, 2, hd), torch.randn(n, 2, hd)
    pos = torch.arange(n)
    full = pm.attention(q, k, v, pos, pos, 0.5)
    assert torch.allclose(full[0], v[0].repeat_interleave(2, 0))              # causal: row 0 sees key 0
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0
    assert torch.allclose(pm.attention(q, k2, v2, pos, pos, 0.5)[:4], full[:4])   # no look-ahead
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    v3 = v.clone(); v3[:, 1] += 1.0
    shifted = pm.attention(q, k, v3, pos, pos, 0.5)
    assert torch.allclose(shifted[:, :2], full[:, :2]) and torch.allclose(shifted[:, 2:], full[:, 2:] + 1.0, atol=1e-6)
    # window 2: query i sees keys i-1 and i only (masked when i >= j + window)
    win = pm.attention(q, k, v, pos, pos, 0.5, window=2)
    ref = pm.attention(q[3:4], k[2:4], v[2:4], pos[3:4], pos[2:4], 0.5)
    assert torch.allclose(win[3:4], ref, atol=1e-6)
    assert torch.allclose(win[:2], full[:2], atol=1e-6)


def test_silu_and_mlp():
    x = torch.tensor([-100.0, -1.0, 0.0, 1.0, 100.0])
    y = pm.silu(x)
    assert float(y[2]) == 0.0 and abs(float(y[3]) - 0.7310586) < 1e-6 and float(y[4]) == 100.0
    assert abs(float(y[0])) < 1e-30
    f = torch.randn(3, 8)
    wg, wu, wd = torch.randn(12, 8), torch.randn(12, 8), torch.randn(8, 12)
    ref = (torch.nn.functional.silu(f @ wg.t()) * (f @ wu.t())) @ wd.t()
    assert torch.allclose(pm.swiglu_mlp(f, wg, wu, wd), ref, atol=1e-4)


def test_forward_is_causal_and_exact_in_prefixes(oracles):
    for name in TINY:
        cfg, tensors = oracles[name]
        (p,) = prompts_for(name, [48])
        whole = pm.forward(cfg, tensors, p)
        assert whole.shape == (48, cfg["vocab_size"])
        part = pm.forward(cfg, tensors, p[:20])
        assert pm.rel_err(part, whole[:20]) < 1e-5
        d64 = pm.forward(cfg, tensors, p, dtype=torch.float64)
        assert pm.rel_err(whole, d64.float()) < 1e-5


def test_window_changes_only_far_rows(oracles):
    cfg, tensors = oracles["C"]                    # layers 2, 3 see the last 40 keys
    (p,) = prompts_for("C", [90])
    win = pm.forward(cfg, tensors, p)
    full = pm.forward(dict(cfg, use_sliding_window=False), tensors, p)
    assert pm.rel_err(win[:40], full[:40]) < 1e-6  # rows 0..39 see every key either way
    assert pm.rel_err(win[40:], full[40:]) > 1e-4


def test_schedule_repeat_and_shared_cache(oracles):
    cfg, tensors = oracles["A"]
    (p,) = prompts_for("A", [12])
    base = pm.forward(cfg, tensors, p)
    assert pm.rel_err(pm.forward(cfg, tensors, p, schedule=[(0, None), (1, None)]), base) == 0.0
    twice = pm.forward(cfg, tensors, p, schedule=[(0, None), (1, None), (1, None)])
    shared = pm.forward(cfg, tensors, p, schedule=[(0, None), (1, None), (1, 1)])
    assert pm.rel_err(twice, base) > 1e-3 and pm.rel_err(shared, twice) > 1e-4


def test_greedy_generate_stops(oracles):
    cfg, tensors = oracles["A"]
    (p,) = prompts_for("A", [5])
    out = pm.greedy_generate(cfg, tensors, p, 6)
    assert len(out) == 6
    cut = pm.greedy_generate(cfg, tensors, p, 6, stop_tokens=[out[2]])
    assert cut == out[:out.index(out[2]) + 1]


# ------------------------------------------------------------------------------- sampling


def test_philox_known_answer():
    assert ps.philox4x32_10([0, 0, 0, 0], 0) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert ps.philox4x32_10([1, 0, 0, 0], 0) != ps.philox4x32_10([0, 0, 0, 0], 0)
    assert ps.philox4x32_10([0, 0, 5, 0], 1 << 40) != ps.philox4x32_10([0, 0, 5, 0], 0)


def test_greedy_is_first_maximum():
    x = np.array([0.1, 3.0, -1.0, 3.0, 2.0], dtype=np.float32)
    assert ps.sample_token(x, ps.Params(), 0) == 1
    assert ps.sample_token(x, ps.Params(temperature=0.0, top_k=1, seed=9), 5) == 1


def test_filters_keep_the_reference_survivors():
    z = np.array([5.0, 4.0, 3.0, 1.0, -40.0], dtype=np.float32)
    c = ps.select_candidates(z, ps.Params(temperature=1.0), [])
    assert [i for i, _ in c] == [0, 1, 2, 3, 4]
    kept = lambda **kw: [i for i, _ in ps.filter_candidates(c, ps.Params(temperature=1.0, **kw))]
    assert kept() == [0, 1, 2, 3]                          # 45 below the maximum: outside the window
    assert kept(top_k=2) == [0, 1]
    assert kept(min_p=0.2) == [0, 1]                       # e^-1 = 0.37 stays, e^-2 = 0.135 goes
    assert kept(top_p=0.6) == [0]                          # p0 = 0.66 reaches 0.6 at once
    assert kept(top_p=0.7) == [0, 1]
    assert kept(top_p=0.999) == [0, 1, 2, 3]
    assert kept(top_k=3, top_p=0.95) == [0, 1, 2]


def test_candidate_cap_and_tie_order():
    z = np.zeros(1000, dtype=np.float32)
    c = ps.select_candidates(z, ps.Params(temperature=0.5), [])
    assert [i for i, _ in c] == list(range(256))           # ties toward the lower id, 256 kept
    z[700] = 1.0
    assert ps.select_candidates(z, ps.Params(temperature=0.5), [])[0] == (700, 2.0)


def test_penalties():
    x = np.array([2.0, -2.0, 1.0, 0.5], dtype=np.float32)
    p = ps.Params(repeat_penalty=2.0, presence_penalty=0.25, frequency_penalty=0.5, repeat_last_n=3)
    out = ps.apply_penalties(x, p, [3, 0, 1, 1])           # window: 0, 1, 1
    assert out.tolist() == [2.0 / 2 - 0.75, -2.0 * 2 - 1.25, 1.0, 0.5]
    assert ps.apply_penalties(x, ps.Params(repeat_last_n=0, repeat_penalty=2.0), [0]).tolist() == x.tolist()
    assert ps.sample_token(x, p, 0, [3, 0, 1, 1]) == 2


def test_draw_is_seeded_and_follows_the_distribution():
    z = np.log(np.array([0.6, 0.3, 0.1], dtype=np.float32))
    p = ps.Params(temperature=1.0, seed=12)
    draws = [ps.sample_token(z, p, pos) for pos in range(3000)]
    assert draws == [ps.sample_token(z, p, pos) for pos in range(3000)]
    assert draws[:50] != [ps.sample_token(z, ps.Params(temperature=1.0, seed=13), pos) for pos in range(50)]
    freq = np.bincount(draws, minlength=3) / 3000.0
    assert np.abs(freq - [0.6, 0.3, 0.1]).max() < 0.03
