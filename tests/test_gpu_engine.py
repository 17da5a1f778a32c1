"""The engine against the plain implementation, in float32 and in bfloat16: each request alone
and whole; with its last 32 tokens one by one; in batches of unequal lengths whose shorter
requests end earlier, one batch after another so that slots are used again; long decoding; the
first tokens of a sequence."""
import pytest
import torch

import plain_model as pm
from conftest import BF16_TOL, FP32_TOL, TINY, check_err, prompts_for, tol
from gpu_util import batch_unequal, engine_for, oracle_logits, tail_one_by_one, whole

pytestmark = pytest.mark.gpu
TOL = {"float32": FP32_TOL, "bfloat16": BF16_TOL}
LENGTHS = {"A": [5, 11, 17, 90], "B": [1, 7, 33, 64, 100], "C": [3, 40, 41, 65, 130, 200],
           "D": [1, 7, 33, 64, 100]}
CASES = [(n, d) for n in TINY for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_each_request_alone_and_whole(model_dirs, oracles, name, dtype):
    eng = engine_for(model_dirs, name, dtype)
    for p in prompts_for(name, LENGTHS[name]):
        check_err(name, dtype, pm.rel_err(whole(eng, p), oracle_logits(oracles, name, p)), f"whole, length {len(p)}")
    eng.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_tokens_one_by_one(model_dirs, oracles, name, dtype):
    eng = engine_for(model_dirs, name, dtype)
    for p in prompts_for(name, [33, LENGTHS[name][-1]], seed=1):
        ref = oracle_logits(oracles, name, p)
        got = tail_one_by_one(eng, p, 32)
        check_err(name, dtype, pm.rel_err(got, ref), f"last 32 one by one, length {len(p)}")
        if dtype == "float32":     # cutting changes nothing beyond rounding
            assert pm.rel_err(got, whole(eng, p)) < FP32_TOL


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_one_after_another(model_dirs, oracles, name, dtype):
    lengths = LENGTHS[name]
    cache_tokens = sum((n + 63) // 64 * 64 for n in lengths)
    eng = engine_for(model_dirs, name, dtype, max_tokens=cache_tokens)   # exactly what one batch holds
    seen_slots = []
    for round_ in range(3):                                              # slots and pages are used again
        reqs = prompts_for(name, lengths[::-1] if round_ % 2 else lengths, seed=10 + round_)
        prompt_lens = [max(1, len(r) - (3 + 5 * i)) for i, r in enumerate(reqs)]
        before = set(eng.cache.records)
        got = batch_unequal(eng, reqs, prompt_lens)
        assert not eng.cache.records and before == set()
        for r, g in zip(reqs, got):
            check_err(name, dtype, pm.rel_err(g, oracle_logits(oracles, name, r)),
                      f"unequal batch, round {round_}, length {len(r)}")
        eng.cache.check()
    assert all(g.pool.free_count == g.pool.n for g in eng.cache.groups)


@pytest.mark.parametrize("name,dtype", CASES)
def test_long_decoding(model_dirs, oracles, name, dtype):
    n = TINY[name]["max_position_embeddings"] if name != "C" else 300
    eng = engine_for(model_dirs, name, dtype)
    (p,) = prompts_for(name, [n], seed=2)
    got = tail_one_by_one(eng, p, n - 4)           # 4 prompt tokens, everything else decoded
    check_err(name, dtype, pm.rel_err(got, oracle_logits(oracles, name, p)), "long decoding")
    # the worst single position, to show where an error would sit (page edges: 64, 128, ...)
    ref = oracle_logits(oracles, name, p)
    per_pos = (got - ref).abs().amax(dim=1) / ref.abs().max()
    assert float(per_pos.max()) < tol(name, dtype), f"worst position {int(per_pos.argmax())}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_context(tmp_path, dtype):
    """Two requests of 1,800 and 700 tokens (29 and 11 cache pages) on configuration B with
    room for 2,048 positions: the prompts in one step, the last 24 tokens of each one by one,
    together in a batch.  In bfloat16 the prompt runs the tensor-memory attention over many
    pages and query tiles, and decoding merges several key splits per request, a different
    number for each."""
    import sonicboom_b200 as sb
    from conftest import INIT
    sb.write_random_model(tmp_path, dict(TINY["B"], max_position_embeddings=2048), seed=21, **INIT["B"])
    cfg, tensors = pm.read_model_dir(tmp_path)
    eng = engine_for({"B": tmp_path}, "B", dtype)
    reqs = prompts_for("B", [1800, 700], seed=6)
    got = batch_unequal(eng, reqs, [len(r) - 24 for r in reqs])
    for r, g in zip(reqs, got):
        ref = pm.forward(cfg, tensors, r)
        per_pos = (g - ref).abs().amax(dim=1) / ref.abs().max()
        check_err("B", dtype, per_pos.max(), f"long context, length {len(r)}, worst position {int(per_pos.argmax())}")
    from sonicboom_b200 import ops
    assert ops.tc5_status() == 0 and ops.attention_status(TINY["B"]["head_dim"]) == 0


def test_a_norm_computed_with_the_product_before_it_changes_nothing(tmp_path, monkeypatch):
    """A wider configuration (8 heads of 64, intermediate 1,024), so that the kernel that adds
    the split o and down products also norms their rows in decoding.  With that hand-over
    switched off (every norm a kernel of its own) the logits agree to float32 rounding: the
    operands of every product differ by at most an ulp of bfloat16 in a few elements."""
    import sonicboom_b200 as sb
    from sonicboom_b200 import ops
    from sonicboom_b200.parts.base import StepContext
    cfg = dict(TINY["B"], hidden_size=256, num_attention_heads=8, num_key_value_heads=2,
               intermediate_size=1024)
    sb.write_random_model(tmp_path, cfg, seed=5, std=0.05)
    eng = engine_for({"W": tmp_path}, "W", "bfloat16")
    reqs = prompts_for("B", [40, 9], seed=8)
    used = []
    real = ops.lib().sb_gemm_tc5_fuses_norm

    def spy(*a):
        used.append(bool(real(*a)))
        return real(*a)
    monkeypatch.setattr(ops.lib(), "sb_gemm_tc5_fuses_norm", spy, raising=False)
    handed = batch_unequal(eng, reqs, [len(r) - 6 for r in reqs])
    assert any(used)
    monkeypatch.setattr(StepContext, "take_normed", lambda self, norm, x: None)
    plain = batch_unequal(eng, reqs, [len(r) - 6 for r in reqs])
    for h, p_ in zip(handed, plain):
        assert pm.rel_err(h, p_) < 2e-3
    pcfg, tensors = pm.read_model_dir(tmp_path)
    for r, h in zip(reqs, handed):
        assert pm.rel_err(h, pm.forward(pcfg, tensors, r)) < BF16_TOL
    assert ops.tc5_status() == 0


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens_of_a_sequence(model_dirs, oracles, name, dtype):
    eng = engine_for(model_dirs, name, dtype)
    reqs = prompts_for(name, [6, 6, 6], seed=3)
    got = batch_unequal(eng, reqs, [1, 2, 1])       # decoding starts right after the first token
    for r, g in zip(reqs, got):
        ref = oracle_logits(oracles, name, r)
        check_err(name, dtype, pm.rel_err(g, ref), "first tokens")
        assert pm.rel_err(g[:2], ref[:2]) < tol(name, dtype) * float(ref.abs().max() / ref[:2].abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_position_and_neighbours_do_not_matter(model_dirs, dtype):
    """A request's logits are the same alone, first, last or in the middle of a batch."""
    eng = engine_for(model_dirs, "B", dtype)
    reqs = prompts_for("B", [70, 9, 33], seed=4)
    alone = [whole(eng, r) for r in reqs]
    for order in ([0, 1, 2], [2, 0, 1], [1, 2, 0]):
        got = batch_unequal(eng, [reqs[i] for i in order], [len(reqs[i]) for i in order])
        for i, g in zip(order, got):
            assert pm.rel_err(g, alone[i]) < (1e-6 if dtype == "float32" else tol("B", dtype)), (order, i)


def test_refusals_reach_the_caller(model_dirs):
    from sonicboom_b200 import StepError
    from sonicboom_b200.cache import CacheFull
    eng = engine_for(model_dirs, "A", "float32", max_tokens=128)
    s = eng.open()
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([(s, [256], [0])])
    with pytest.raises(StepError, match="max_position_embeddings"):
        eng.step([(s, [1] * 129, [])])
    t = eng.open()
    eng.step([(s, [1] * 100, [])])
    with pytest.raises(CacheFull):
        eng.step([(t, [1] * 10, [])])
    assert eng.step([(s, [2], [])]) is None


# --------------------------------------------------- two layers with the sizes of a 7B model
BIG = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=3584,
           num_hidden_layers=2, num_attention_heads=28, num_key_value_heads=4,
           intermediate_size=18944, vocab_size=8192, rope_theta=1000000.0, rms_norm_eps=1e-6,
           max_position_embeddings=16384, tie_word_embeddings=False)
BIG_INIT = dict(std=0.02, bias_std=0.02, norm_std=0.05)
BIG_SEED = 3


@pytest.fixture(scope="module")
def big_models():
    """The same seeded weights as a float32 and as a bfloat16 model (the random tensors are a
    function of seed, name and index, rounded to bfloat16 before either model sees them)."""
    import sonicboom_b200 as sb
    models = {d: sb.random_model(BIG, BIG_SEED, dtype=d, device="cuda:0", **BIG_INIT)
              for d in ("float32", "bfloat16")}
    yield models
    models.clear()
    torch.cuda.empty_cache()


def big_requests(lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, BIG["vocab_size"], (n,), generator=g).tolist() for n in lengths]


def test_float32_path_against_the_plain_implementation_at_7b_layer_sizes(big_models):
    """Width 3,584, 28/4 heads of 128, intermediate 18,944: the true 32-bit path against the
    plain implementation on a 256-token request (whole, and with its last 32 tokens one by
    one), on the same random tensors, which the plain side gets from the generator's device
    form copied to the host."""
    import sonicboom_b200 as sb
    from sonicboom_b200.models import tensor_requests
    from sonicboom_b200.weights import RandomSource
    src = RandomSource(tensor_requests(big_models["float32"].spec), BIG_SEED, device="cuda:0", **BIG_INIT)
    tensors = {n: src.tensor(n).float().cpu() for n in src.names()}
    (req,) = big_requests([256], seed=5)
    ref = pm.forward(BIG, tensors, req, dtype=torch.float64).float()   # sums of 18,944 terms: the
    eng = sb.Engine(big_models["float32"], max_tokens=512)             # oracle itself must not round
    check_err("7B", "float32", pm.rel_err(whole(eng, req), ref), "whole, 256 tokens")
    check_err("7B", "float32", pm.rel_err(tail_one_by_one(eng, req, 32), ref), "last 32 one by one")


def test_bfloat16_path_against_the_float32_path_at_7b_layer_sizes(big_models):
    """The serving path (tcgen05 products, tensor-memory and split attention, fused norms)
    against the engine's own float32 path on the same weights: a request whole, with its last
    32 tokens one by one, and in an unequal batch of three whose shorter requests end earlier.
    The three cuts of the bfloat16 path are also held against each other."""
    import sonicboom_b200 as sb
    from sonicboom_b200 import ops
    e32 = sb.Engine(big_models["float32"], max_tokens=4096)
    e16 = sb.Engine(big_models["bfloat16"], max_tokens=4096)
    reqs = big_requests([1100, 300, 70], seed=6)
    tail = 32
    want = lambda r: list(range(len(r) - tail, len(r)))     # the last 32 positions' logits

    def whole_tail(eng, r):
        s = eng.open()
        out = eng.step([(s, r, want(r))]).float().cpu()
        eng.close(s)
        return out

    refs = [whole_tail(e32, r) for r in reqs]
    for r, ref in zip(reqs, refs):
        check_err("7B", "bfloat16", pm.rel_err(whole_tail(e16, r), ref), f"whole, length {len(r)}")
        got = tail_one_by_one(e16, r, tail)[-tail:]
        check_err("7B", "bfloat16", pm.rel_err(got, ref), f"last 32 one by one, length {len(r)}")
    got = batch_unequal(e16, reqs, [len(r) - tail - 5 * i for i, r in enumerate(reqs)])
    for r, g, ref in zip(reqs, got, refs):
        check_err("7B", "bfloat16", pm.rel_err(g[-tail:], ref), f"unequal batch, length {len(r)}")
    # and the float32 path's own cuts agree with each other far more closely
    got32 = batch_unequal(e32, reqs[1:], [len(r) - tail for r in reqs[1:]])
    for g, ref in zip(got32, refs[1:]):
        check_err("7B", "float32", pm.rel_err(g[-tail:], ref), "float32 cuts against each other")
    assert ops.tc5_status() == 0 and ops.attention_status(128) == 0


def test_layers_of_a_7b_model_decode_as_they_prefill():
    """Two layers with the sizes of a 7B model (width 3,584, 28/4 heads of 128, intermediate
    18,944) and requests of 8,224 and 3,032 tokens: whole in one step, and with the last 32
    tokens one by one in a batch of two.  The prompt runs the persistent tcgen05 products and
    the tensor-memory attention over 129 pages; decoding runs the split products with the norm
    in their reduce kernel, and key splits of 512 (the long request) and 256 (the short one).
    No oracle at this size: the two cuts are held against each other."""
    import sonicboom_b200 as sb
    from sonicboom_b200 import ops
    cfg = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=3584,
               num_hidden_layers=2, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, vocab_size=32000, rope_theta=1000000.0, rms_norm_eps=1e-6,
               max_position_embeddings=16384, tie_word_embeddings=False)
    model = sb.random_model(cfg, seed=3, dtype="bfloat16", device="cuda:0", std=0.02)
    eng = sb.Engine(model, max_tokens=16384)
    g = torch.Generator().manual_seed(11)
    reqs = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (8224, 3032)]
    tail = 32
    slots = [eng.open() for _ in reqs]
    whole = eng.step([(s, r, list(range(len(r) - tail, len(r)))) for s, r in zip(slots, reqs)]).float().cpu()
    for s in slots:
        eng.close(s)
    slots = [eng.open() for _ in reqs]
    assert eng.step([(s, r[:-tail], []) for s, r in zip(slots, reqs)]) is None
    steps = [eng.step([(s, [r[len(r) - tail + t]], [0]) for s, r in zip(slots, reqs)]).float().cpu()
             for t in range(tail)]
    for s in slots:
        eng.close(s)
    for i in range(len(reqs)):
        cut = torch.stack([st[i] for st in steps])
        ref = whole[i * tail:(i + 1) * tail]
        per_pos = (cut - ref).abs().amax(dim=1) / ref.abs().max()
        assert float(per_pos.max()) < BF16_TOL, f"request {i}: worst position {int(per_pos.argmax())}"
    assert ops.tc5_status() == 0 and ops.attention_status(128) == 0
    del eng, model
    torch.cuda.empty_cache()
