"""Generation through the entry points: greedy against the plain implementation, sampling
against the plain sampler, sessions, the command line, and trace replay as a program."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_model as pm
import plain_sampling as ps
from conftest import BF16_TOL, FP32_TOL, ROOT, TINY, check_err, prompts_for
from sonicboom_b200 import llm
from sonicboom_b200.sampling import Sampling

pytestmark = pytest.mark.gpu
TOL = {"float32": FP32_TOL, "bfloat16": BF16_TOL}


def plain_tokens(oracle, prompt, n, sampling: Sampling = None, stops=()):
    """Continuation by whole-sequence forwards of the plain model and the plain sampler;
    also returns each step's margin between the two best adjusted scores."""
    cfg, tensors = oracle
    seq, out, margins = list(prompt), [], []
    s = sampling or Sampling()
    p = ps.Params(s.temperature, s.top_k, s.top_p, s.min_p, s.seed, s.repeat_penalty, s.repeat_last_n,
                  s.presence_penalty, s.frequency_penalty)
    for _ in range(n):
        logits = pm.forward(cfg, tensors, seq)[-1].numpy()
        top2 = np.sort(logits)[-2:]
        margins.append(float(top2[1] - top2[0]))
        tok = ps.sample_token(logits, p, len(seq), seq)
        out.append(tok); seq.append(tok)
        if tok in stops:
            break
    return out, margins


def assert_same_or_near_tie(got, want, margins, scale, dtype):
    """Tokens agree; the first difference is allowed only where the two best scores are
    closer than the dtype's tolerance (the reference's near-tie rule, docs/benchmark.md:263-266)."""
    for i, (g, w) in enumerate(zip(got, want)):
        if g != w:
            assert dtype == "bfloat16" and margins[i] < 2 * BF16_TOL * scale, (i, got, want, margins[i])
            return
    assert len(got) == len(want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_of_a_batch(model_dirs, oracles, name, dtype):
    model = llm.model_load(model_dirs[name], dtype=dtype)
    assert model.arch == "Qwen2ForCausalLM" and model.vocab_size == TINY[name]["vocab_size"]
    lens = {"A": [5, 11, 17], "B": [1, 7, 33, 64, 100], "C": [3, 50, 70], "D": [1, 7, 33, 64, 100]}[name]
    n_new = {"A": 8, "B": 16, "C": 12, "D": 16}[name]
    prompts = prompts_for(name, lens, seed=5)
    outs = llm.generate_batch(model, prompts, max_tokens=n_new, ignore_eos=True)
    scale = float(pm.forward(*oracles[name], prompts[0]).abs().max())
    for p, o in zip(prompts, outs):
        want, margins = plain_tokens(oracles[name], p, n_new)
        assert_same_or_near_tie(o, want, margins, scale, dtype)
    # each sequence alone gives what it gave in the batch, and a small cache means more batches
    alone = [llm.generate_batch(model, [p], max_tokens=n_new, ignore_eos=True)[0] for p in prompts]
    small = llm.generate_batch(model, prompts, max_tokens=n_new, ignore_eos=True,
                               max_cache_tokens=max((len(p) + n_new + 63) // 64 * 64 for p in prompts) + 64)
    if dtype == "float32":
        assert alone == outs and small == outs


def test_dependent_launch_changes_no_token(model_dirs):
    """The kernels of a step may overlap through programmatic dependent launch; with it off,
    on for the default kernel classes, and on for every kernel the same tokens come out
    bit for bit (each kernel waits before it touches what a predecessor wrote), and no bounded
    wait of the tensor-memory kernels gives up."""
    from sonicboom_b200 import ops
    model = llm.model_load(model_dirs["B"], dtype="bfloat16")
    prompts = prompts_for("B", [3, 40, 90, 129], seed=9)
    default = ops.lib().sb_pdl_enabled()
    outs = {}
    try:
        for mask in (0, default, ops.PDL_ALL):
            ops.set_pdl(mask)
            outs[mask] = llm.generate_batch(model, prompts, max_tokens=24, ignore_eos=True)
    finally:
        ops.set_pdl(default)
    assert outs[0] == outs[default] == outs[ops.PDL_ALL]
    if "SB_PDL" not in os.environ:
        assert default == ops.PDL_ALL & ~ops.PDL_SKINNY
    assert ops.tc5_status() == 0 and ops.attention_status(TINY["B"]["head_dim"]) == 0


def test_trace_ranges_change_no_token(model_dirs):
    """With the opt-in NVTX ranges on (per step, per schedule entry, per captured decode step)
    the same tokens come out."""
    from sonicboom_b200 import ops
    model = llm.model_load(model_dirs["B"], dtype="bfloat16")
    prompts = prompts_for("B", [3, 40, 90], seed=15)
    off = llm.generate_batch(model, prompts, max_tokens=12, ignore_eos=True)
    ops.set_trace(True)
    try:
        on = llm.generate_batch(model, prompts, max_tokens=12, ignore_eos=True)
    finally:
        ops.set_trace(False)
    assert on == off


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stop_tokens_and_eos(model_dirs, oracles, dtype):
    model = llm.model_load(model_dirs["A"], dtype=dtype)
    assert model.eos == (7,)
    prompts = prompts_for("A", [5, 11, 17], seed=6)
    free = llm.generate_batch(model, prompts, max_tokens=10, ignore_eos=True)
    stop = free[1][3]
    outs = llm.generate_batch(model, prompts, max_tokens=10, stop_tokens=[stop])
    for f, o in zip(free, outs):
        cut = f.index(stop) + 1 if stop in f else len(f)
        assert o == f[:cut]                        # the stop token is emitted, then the sequence ends
    assert outs[1][-1] == stop and len(outs[1]) <= 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_budgets_next_to_the_context_limit(model_dirs, oracles, dtype):
    """Configuration A holds 128 positions.  Prompts of 100, 5 and 5 tokens that may produce 20,
    100 and 100: the first request is finished after 20 tokens and stays a row of the captured
    batch while the others go on for 80 more steps.  It must stay inside its own two pages:
    the others' tokens are what they are alone, and what the plain implementation gives."""
    model = llm.model_load(model_dirs["A"], dtype=dtype)
    prompts = prompts_for("A", [100, 5, 5], seed=12)
    per = [Sampling(max_tokens=m) for m in (20, 100, 100)]
    outs = llm.generate_batch(model, prompts, sampling=per, ignore_eos=True)
    assert [len(o) for o in outs] == [20, 100, 100]
    scale = float(pm.forward(*oracles["A"], prompts[0]).abs().max())
    for p, s, o in zip(prompts, per, outs):
        alone = llm.generate_batch(model, [p], sampling=s, ignore_eos=True)[0]
        want, margins = plain_tokens(oracles["A"], p, s.max_tokens)
        if dtype == "float32":
            assert o == alone == want
        else:
            assert_same_or_near_tie(o, want, margins, scale, dtype)
            assert_same_or_near_tie(alone, want, margins, scale, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_cache_of_exactly_what_the_batch_was_admitted_for(model_dirs, oracles, dtype):
    """Four requests with budgets 3, 150, 4 and 40 in a cache of exactly the pages their prompts
    and own budgets need (1 + 3 + 1 + 1): the captured loop reserves each row's own budget, is
    captured again when half of the rows have finished, and the engine ends with every page and
    slot free."""
    from sonicboom_b200 import Engine
    model = llm.model_load(model_dirs["B"], dtype=dtype)
    prompts = prompts_for("B", [10, 12, 30, 7], seed=13)
    per = [Sampling(max_tokens=m) for m in (3, 150, 4, 40)]
    engine = Engine(model.decoder, max_tokens=64 * 6)
    outs = llm.generate_batch(model, prompts, sampling=per, ignore_eos=True, engine=engine)
    assert [len(o) for o in outs] == [3, 150, 4, 40]
    engine.cache.check()
    assert not engine.cache.records and engine.free_pages() == 6
    scale = float(pm.forward(*oracles["B"], prompts[2]).abs().max())
    for p, s, o in zip(prompts, per, outs):
        want, margins = plain_tokens(oracles["B"], p, s.max_tokens)
        if dtype == "float32":
            assert o == want
        else:
            assert_same_or_near_tie(o, want, margins, scale, dtype)
    # one page less and the batch is two batches; the tokens stay the same in float32
    small = Engine(model.decoder, max_tokens=64 * 5)
    again = llm.generate_batch(model, prompts, sampling=per, ignore_eos=True, engine=small)
    if dtype == "float32":
        assert again == outs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_windowed_model_decodes_through_the_captured_loop(model_dirs, oracles, dtype, monkeypatch):
    """Configuration C has layers with a window of 40 keys.  Its decode steps are captured like
    any other model's: the windowed group holds its pages while the loop lives and gives back
    the ones behind the window when the loop is closed.  Same tokens as step by step without
    the captured loop, and as the plain implementation."""
    from sonicboom_b200 import Engine
    from sonicboom_b200.engine.decode import DecodeLoop
    model = llm.model_load(model_dirs["C"], dtype=dtype)
    made = []
    real_init = DecodeLoop.__init__

    def spy(self, *a, **k):
        real_init(self, *a, **k)
        made.append(self)
    monkeypatch.setattr(DecodeLoop, "__init__", spy)
    prompts = prompts_for("C", [3, 50, 70], seed=14)
    per = [Sampling(max_tokens=m) for m in (90, 30, 100)]
    engine = Engine(model.decoder, max_tokens=64 * 8)
    outs = llm.generate_batch(model, prompts, sampling=per, ignore_eos=True, engine=engine)
    assert made and any(g.need.window > 0 for g in engine.cache.groups)
    engine.cache.check()
    assert not engine.cache.records and engine.free_pages() == 8
    stepwise = Engine(model.decoder, max_tokens=64 * 8)
    stepwise.use_decode_loop = False
    n_loops = len(made)
    again = llm.generate_batch(model, prompts, sampling=per, ignore_eos=True, engine=stepwise)
    assert len(made) == n_loops
    scale = float(pm.forward(*oracles["C"], prompts[1]).abs().max())
    for p, s, o, a in zip(prompts, per, outs, again):
        want, margins = plain_tokens(oracles["C"], p, s.max_tokens)
        if dtype == "float32":
            assert o == a == want
        else:
            assert_same_or_near_tie(o, want, margins, scale, dtype)
            assert_same_or_near_tie(a, want, margins, scale, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sampled_generation_matches_the_plain_sampler(model_dirs, oracles, dtype):
    model = llm.model_load(model_dirs["A"], dtype=dtype)
    prompts = prompts_for("A", [5, 11, 17], seed=7)
    s = Sampling(temperature=0.8, seed=1234, max_tokens=8)
    outs = llm.generate_batch(model, prompts, sampling=s, ignore_eos=True)
    again = llm.generate_batch(model, prompts[::-1], sampling=s, ignore_eos=True)[::-1]
    assert outs == again                           # the row in the batch does not matter
    other = llm.generate_batch(model, prompts, sampling=Sampling(temperature=0.8, seed=1235, max_tokens=8),
                               ignore_eos=True)
    assert other != outs
    if dtype == "float32":
        for p, o in zip(prompts, outs):
            want, _ = plain_tokens(oracles["A"], p, 8, s)
            assert o == want
    rich = Sampling(temperature=1.1, top_k=20, top_p=0.9, min_p=0.02, seed=5, max_tokens=8,
                    repeat_penalty=1.2, presence_penalty=0.1, frequency_penalty=0.1, repeat_last_n=8)
    outs = llm.generate_batch(model, prompts, sampling=rich, ignore_eos=True)
    if dtype == "float32":
        for p, o in zip(prompts, outs):
            assert o == plain_tokens(oracles["A"], p, 8, rich)[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_session_prefill_decode_and_prefix_reuse(model_dirs, oracles, dtype):
    model = llm.model_load(model_dirs["B"], dtype=dtype)
    (p,) = prompts_for("B", [40], seed=8)
    sess = llm.session_new(model, 256)
    assert sess.prefill(p) == 0
    seen = []
    first = sess.decode(Sampling(max_tokens=5), cb=lambda t: seen.append(t) or 0)
    more = sess.decode(Sampling(max_tokens=4))      # decode continues where it stopped
    assert seen == first and len(more) == 4
    whole = llm.generate_tokens(llm.session_new(model, 256), p, 9)
    assert whole == first + more
    if dtype == "float32":
        assert whole == plain_tokens(oracles["B"], p, 9)[0]
    # a new prompt that shares 24 tokens with the old one reuses them; the result is the same
    p2 = p[:24] + prompts_for("B", [16], seed=9)[0]
    reused = sess.prefill(p2)
    assert reused == 24
    cont = sess.decode(Sampling(max_tokens=6))
    fresh = llm.generate_tokens(llm.session_new(model, 256), p2, 6)
    assert cont == fresh
    assert sess.prefill(p2) == len(p2) - 1          # the last prompt token is always processed
    stopped = sess.decode(Sampling(max_tokens=6), cb=lambda t: 1)
    assert stopped == fresh[:1]
    with pytest.raises(ValueError, match="n_ctx"):
        sess.prefill([1] * 300)


def test_command_line(model_dirs, tmp_path):
    tokens = tmp_path / "prompts.txt"
    prompts = prompts_for("A", [5, 11], seed=10)
    tokens.write_text("\n".join(" ".join(map(str, p)) for p in prompts) + "\n")
    cmd = [sys.executable, str(ROOT / "bin" / "sonicboom_b200"), "generate", "-m", str(model_dirs["A"]),
           "--tokens", str(tokens), "-n", "6", "--dtype", "float32", "--ignore-eos"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [[int(t) for t in l.split()] for l in r.stdout.strip().splitlines()]
    model = llm.model_load(model_dirs["A"], dtype="float32")
    assert lines == llm.generate_batch(model, prompts, max_tokens=6, ignore_eos=True)
    r = subprocess.run(cmd + ["--temperature", "0.9", "--seed", "3", "--top-k", "10"],
                       capture_output=True, text=True, timeout=600)
    sampled = [[int(t) for t in l.split()] for l in r.stdout.strip().splitlines()]
    assert sampled == llm.generate_batch(model, prompts, max_tokens=6, ignore_eos=True, temperature=0.9,
                                         seed=3, top_k=10)


# ----------------------------------------------------------------------------- trace replay

def replay(model_dir, dtype, steps, out_dir, max_tokens):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                        "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                       input=text, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    return {int(p.stem): np.fromfile(p, dtype="<f4") for p in Path(out_dir).glob("*.f32")}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C", "D"])
def test_trace_replay_three_cuts(model_dirs, oracles, tmp_path, name, dtype):
    vocab = TINY[name]["vocab_size"]
    reqs = {f"r{i}": p for i, p in enumerate(prompts_for(name, [100, 40, 70], seed=11))}
    refs = {k: pm.forward(*oracles[name], v).numpy() for k, v in reqs.items()}
    # (1) each request alone and whole; (2) the last 32 tokens one by one; (3) two batches of
    # unequal lengths one after the other in a cache that holds only one of them at a time
    steps, expect = [], {}
    n = 0
    for k, v in reqs.items():
        steps.append({"step": n, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))}], "end": [k]})
        expect[n] = refs[k]
        n += 1
    for k, v in reqs.items():
        cut = len(v) - 32
        steps.append({"step": n, "entries": [{"id": k + "x", "tokens": v[:cut], "want": [cut - 1]}], "end": []})
        expect[n] = refs[k][cut - 1:cut]
        n += 1
        for j in range(cut, len(v)):
            steps.append({"step": n, "entries": [{"id": k + "x", "tokens": [v[j]], "want": [0]}],
                          "end": [k + "x"] if j == len(v) - 1 else []})
            expect[n] = refs[k][j:j + 1]
            n += 1
    for round_ in range(2):
        ids = [f"{k}b{round_}" for k in reqs]
        fed = {i: len(v) - 10 - 7 * j for j, (i, v) in enumerate(zip(ids, reqs.values()))}
        steps.append({"step": n, "entries": [{"id": i, "tokens": v[:fed[i]], "want": [0, fed[i] - 1]}
                                             for i, v in zip(ids, reqs.values())], "end": []})
        expect[n] = np.concatenate([refs[k][[0, fed[i] - 1]] for i, k in zip(ids, reqs)])
        n += 1
        live = dict(zip(ids, reqs))
        while live:
            entries, rows, ends = [], [], []
            for i, k in list(live.items()):
                entries.append({"id": i, "tokens": [reqs[k][fed[i]]], "want": [0] if fed[i] % 2 else []})
                if fed[i] % 2:
                    rows.append(refs[k][fed[i]:fed[i] + 1])
                fed[i] += 1
                if fed[i] == len(reqs[k]):
                    ends.append(i)
                    del live[i]
            steps.append({"step": n, "entries": entries, "end": ends})
            if rows:
                expect[n] = np.concatenate(rows)
            n += 1
    max_tokens = sum((len(v) + 63) // 64 * 64 for v in reqs.values())
    got = replay(model_dirs[name], dtype, steps, tmp_path / "out", max_tokens)
    assert set(got) == set(expect)
    scale = max(float(np.abs(r).max()) for r in refs.values())
    for step_no, ref in expect.items():
        g = got[step_no].reshape(-1, vocab)
        assert g.shape == ref.shape, step_no
        check_err(name, dtype, float(np.abs(g - ref).max()) / scale, f"replay step {step_no}")
    # the index beside the logits names the request and the position of every row written
    index = [json.loads(l) for l in (tmp_path / "out" / "index.jsonl").read_text().splitlines()]
    assert [r["step"] for r in index] == sorted(expect)
    by_step = {r["step"]: r["rows"] for r in index}
    assert by_step[0] == [["r0", i] for i in range(len(reqs["r0"]))]
    last = max(expect)
    assert len(by_step[last]) == expect[last].shape[0] and all(len(r) == 2 for r in by_step[last])
    first_decode = len(reqs) + 1                  # the step after request r0's prefix step
    assert by_step[first_decode] == [["r0x", len(reqs["r0"]) - 32]]
