"""Each part alone against the plain implementation, the run order as data (a layer twice, a
layer reading another's cache), and a toy mixer with state of its own that is registered,
built and stepped without a change to the package; likewise a toy feed-forward that routes
rows to experts and a toy position encoding."""
import dataclasses

import pytest
import torch

import plain_model as pm
import sonicboom_b200 as sb
from conftest import BF16_TOL, FP32_TOL, TINY, prompts_for
from sonicboom_b200 import parts
from sonicboom_b200.cache import Cache, StateNeed
from sonicboom_b200.config import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                                   PositionSpec, ScheduleEntry, spec_from_config_dict)
from sonicboom_b200.engine.step import StepEntry, StepPlan
from sonicboom_b200.models import DecoderModel
from sonicboom_b200.weights import RandomSource, TensorRequest, check, fetch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": FP32_TOL, "bfloat16": BF16_TOL}


def bound(part, tensors, dtype):
    part.bind(lambda n: tensors[n].to(DEV, dtype if tensors[n].is_floating_point() else None))
    return part


def ctx_for(part_needs, lens, dtype):
    cache = Cache(part_needs, [None] * len(part_needs), 4096, dtype, DEV)
    slots = [cache.open() for _ in lens]
    for s, n in zip(slots, lens):
        cache.reserve(s, n)
    plan = StepPlan(cache, [StepEntry(s, [0] * n, []) for s, n in zip(slots, lens)], DEV)
    return parts.StepContext(plan=plan, cache=cache, entry=0, kv_entry=0, owns_cache=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_norm_mixer_feed_forward_and_block_alone(oracles, name, dtype):
    cfg, tensors = oracles[name]
    _, spec = spec_from_config_dict(cfg)
    dt, tol = DT[dtype], (1e-5 if dtype == "float32" else BF16_TOL)
    layer = spec.layers[-1]                       # the last layer is the windowed one in C
    li = len(spec.layers) - 1
    lens = [9, 70]
    x = torch.randn(sum(lens), spec.width, generator=torch.Generator().manual_seed(1))

    norm = bound(parts.make(parts.NORMS, "norm", layer.mixer_norm, dt, DEV), tensors, dt)
    h = norm.forward(x.to(DEV), dt)
    h_ref = pm.rms_norm(x, tensors[layer.mixer_norm.tensor], layer.mixer_norm.eps)
    assert pm.rel_err(h.float().cpu(), h_ref) < (1e-6 if dtype == "float32" else 5e-3)

    pos = parts.make(parts.POSITION_ENCODINGS, "position encoding", layer.mixer.position, dt, DEV)
    i = torch.arange(layer.mixer.head_dim // 2, dtype=torch.float32)
    inv_ref = torch.exp(-2.0 * i / layer.mixer.head_dim * torch.log(torch.tensor(cfg["rope_theta"])))
    assert torch.allclose(pos.inv_freq.cpu(), inv_ref, rtol=1e-6) and pos.rotary_dim == layer.mixer.head_dim

    mixer = bound(parts.make(parts.MIXERS, "mixer", layer.mixer, dt, DEV), tensors, dt)
    ctx = ctx_for([mixer.kv_need()], lens, dt)
    hin = h_ref.to(DEV, dt)
    mixed = mixer.forward(hin, ctx).cpu()
    window = pm.layer_windows(cfg)[li]
    at = 0
    for n in lens:
        ref, _ = pm.self_attention(hin[at:at + n].float().cpu(), torch.arange(n),
                                   f"model.layers.{li}.", cfg, window, tensors)
        assert pm.rel_err(mixed[at:at + n], ref) < tol
        at += n
    res = torch.randn_like(mixed).to(DEV)
    ctx2 = ctx_for([mixer.kv_need()], lens, dt)
    with_res = mixer.forward(hin, ctx2, residual=res.clone()).cpu()
    assert pm.rel_err(with_res, mixed + res.cpu()) < tol
    # an output-projection bias (not this architecture's, but a spec may ask for one)
    biased_spec = dataclasses.replace(layer.mixer, out_bias=True)
    o_bias = torch.randn(spec.width, generator=torch.Generator().manual_seed(3)) * 0.1
    biased = bound(parts.make(parts.MIXERS, "mixer", biased_spec, dt, DEV),
                   dict(tensors, **{layer.mixer.prefix + "o_proj.bias": o_bias}), dt)
    assert any(r.name.endswith("o_proj.bias") for r in biased.tensor_requests())
    ctx4 = ctx_for([mixer.kv_need()], lens, dt)
    with_bias = biased.forward(hin, ctx4, residual=res.clone()).cpu()
    expect = with_res + (o_bias.to(dt).float() if dtype == "bfloat16" else o_bias)
    assert pm.rel_err(with_bias, expect) < (1e-6 if dtype == "float32" else 1e-5)

    ffn = bound(parts.make(parts.FEED_FORWARDS, "feed-forward", layer.feed_forward, dt, DEV), tensors, dt)
    p = f"model.layers.{li}.mlp."
    fed = ffn.forward(hin, ctx).cpu()
    ref = pm.swiglu_mlp(hin.float().cpu(), tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"],
                        tensors[p + "down_proj.weight"])
    assert pm.rel_err(fed, ref) < tol

    block = bound(parts.make(parts.BLOCKS, "block arrangement", layer, dt, DEV), tensors, dt)
    ctx3 = ctx_for([block.kv_need()], lens, dt)
    y = block.forward(x.to(DEV).clone(), ctx3).cpu()
    at = 0
    for n in lens:
        ref, _ = pm.block(x[at:at + n], torch.arange(n), li, cfg, window, tensors)
        assert pm.rel_err(y[at:at + n], ref) < tol
        at += n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_order_is_data(model_dirs, oracles, dtype):
    """A layer named twice runs twice with a cache per run; an entry may read another's cache."""
    cfg, tensors = oracles["B"]
    _, spec = spec_from_config_dict(cfg)
    (p,) = prompts_for("B", [50])
    for schedule in ([(0, None), (1, None), (1, None), (2, None)],
                     [(0, None), (1, None), (2, 1), (2, None), (0, 0)]):
        s2 = dataclasses.replace(spec, schedule=tuple(ScheduleEntry(l, c) for l, c in schedule))
        model = DecoderModel(s2, DT[dtype], DEV)
        src = sb.weights.SafetensorsDir(model_dirs["B"])
        check(src, model.tensor_requests())
        model.bind(lambda n: fetch(src, n, model.dtype, model.device))
        assert [n is None for n in model.kv_needs()] == [c is not None for _, c in schedule]
        eng = sb.Engine(model, max_tokens=512)
        ref = pm.forward(cfg, tensors, p, schedule=schedule)
        s = eng.open()
        got = [eng.step([(s, p[:30], list(range(30)))]).cpu()]
        got += [eng.step([(s, [t], [0])]).cpu() for t in p[30:]]
        assert pm.rel_err(torch.cat(got), ref) < TOL[dtype]


# ----------------------------------------------------------------- a toy mixer with state

class RunningMean(parts.Mixer):
    """out_t = W . mean(h_0..h_t): needs no keys or values, only a running sum and a count
    per sequence, which it keeps in the cache's per-slot state."""

    def __init__(self, spec, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.w = None

    def state_need(self):
        return StateNeed((self.spec.width + 1,), torch.float32)

    def tensor_requests(self):
        return [TensorRequest(self.spec.prefix + "weight", (self.spec.width, self.spec.width))]

    def bind(self, get):
        self.w = get(self.spec.prefix + "weight").float()

    def forward(self, h, ctx, residual=None):
        d = self.spec.width
        state = ctx.state()
        if ctx.plan.n_rows == ctx.plan.n_seqs:
            # one row per sequence (decoding): device work only, so that the step can be
            # captured in a CUDA graph
            slots_dev = ctx.plan.seq_slot.long()
            sums = state[slots_dev, :d] + h.float()
            count = state[slots_dev, d] + 1.0
            state[slots_dev, :d], state[slots_dev, d] = sums, count
            out = (sums / count[:, None]) @ self.w.t()
            return out + residual if residual is not None else out
        row0 = ctx.plan.seq_row0.cpu().tolist()
        slots = ctx.plan.seq_slot.cpu().tolist()
        out = torch.empty(h.shape[0], d, dtype=torch.float32, device=h.device)
        for b, slot in enumerate(slots):
            rows = slice(row0[b], row0[b + 1])
            sums = state[slot, :d] + h[rows].float().cumsum(0)
            count = state[slot, d] + torch.arange(1, sums.shape[0] + 1, device=h.device)
            out[rows] = (sums / count[:, None]) @ self.w.t()
            state[slot, :d], state[slot, d] = sums[-1], count[-1]
        return out + residual if residual is not None else out


def toy_spec(width=48, vocab=97, n_layers=3):
    layers = []
    for i in range(n_layers):
        p = f"toy.layers.{i}."
        if i == 1:
            mixer = MixerSpec(kind="running_mean", width=width, prefix=p + "mix.")
        else:
            mixer = MixerSpec(kind="attention", width=width, n_heads=3, n_kv_heads=1, head_dim=16,
                              scale=0.25, qkv_bias=True, prefix=p + "self_attn.",
                              position=PositionSpec("rope_neox", 16, 5000.0))
        layers.append(LayerSpec("pre_norm", mixer, NormSpec("rmsnorm", width, 1e-5, p + "n1.weight"),
                                FeedForwardSpec("swiglu", width, 64, prefix=p + "mlp."),
                                NormSpec("rmsnorm", width, 1e-5, p + "n2.weight")))
    return ModelSpec("Toy", width, vocab, 256, "toy.embed.weight", tuple(layers),
                     tuple(ScheduleEntry(i) for i in range(n_layers)),
                     NormSpec("rmsnorm", width, 1e-5, "toy.norm.weight"), None)


def toy_reference(tensors, spec, tokens, head=None):
    """Whole-sequence forward of the toy model from plain parts."""
    t = {k: v.float().cpu() for k, v in tensors.items()}
    n = len(tokens)
    pos = torch.arange(n)
    x = pm.embedding(t["toy.embed.weight"], tokens)
    for i, layer in enumerate(spec.layers):
        p = f"toy.layers.{i}."
        h = pm.rms_norm(x, t[p + "n1.weight"], 1e-5)
        if layer.mixer.kind == "running_mean":
            mean = h.cumsum(0) / torch.arange(1, n + 1)[:, None]
            mixed = mean @ t[p + "mix.weight"].t()
        else:
            a = p + "self_attn."
            q = pm.rope_neox(pm.linear(h, t[a + "q_proj.weight"], t[a + "q_proj.bias"]).view(n, 3, 16), pos, 5000.0)
            k = pm.rope_neox(pm.linear(h, t[a + "k_proj.weight"], t[a + "k_proj.bias"]).view(n, 1, 16), pos, 5000.0)
            v = pm.linear(h, t[a + "v_proj.weight"], t[a + "v_proj.bias"]).view(n, 1, 16)
            mixed = pm.linear(pm.attention(q, k, v, pos, pos, 0.25).reshape(n, 48), t[a + "o_proj.weight"])
        x = x + mixed
        f = pm.rms_norm(x, t[p + "n2.weight"], 1e-5)
        x = x + pm.swiglu_mlp(f, t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"],
                              t[p + "mlp.down_proj.weight"])
    head = t["toy.embed.weight"] if head is None else head.float().cpu()
    return pm.linear(pm.rms_norm(x, t["toy.norm.weight"], 1e-5), head)


def toy_reference_with_head(tensors, spec, tokens, head):
    return toy_reference(tensors, spec, tokens, head=head)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_mixer_with_state_registers_builds_and_steps(dtype):
    parts.register_mixer("running_mean", RunningMean)
    try:
        spec = toy_spec()
        model = DecoderModel(spec, DT[dtype], DEV)
        src = RandomSource(model.tensor_requests(), seed=4, std=0.08, bias_std=0.05, norm_std=0.1)
        check(src, model.tensor_requests())
        tensors = {n: src.tensor(n) for n in src.names()}
        model.bind(lambda n: fetch(src, n, model.dtype, model.device))
        assert model.kv_needs()[1] is None and model.state_needs()[1] is not None
        eng = sb.Engine(model, max_tokens=1024)
        assert set(eng.cache.state) == {1} and len(eng.cache.groups) == 1
        g = torch.Generator().manual_seed(0)
        reqs = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (40, 7, 90)]
        for round_ in range(2):                    # the second round reuses slots: state starts at zero
            slots = [eng.open() for _ in reqs]
            cut = [25, 3, 60]
            first = eng.step([(s, r[:c], list(range(c))) for s, r, c in zip(slots, reqs, cut)]).cpu()
            second = eng.step([(s, r[c:], list(range(len(r) - c))) for s, r, c in zip(slots, reqs, cut)]).cpu()
            a = b = 0
            for r, c in zip(reqs, cut):
                ref = toy_reference(tensors, spec, r)
                got = torch.cat([first[a:a + c], second[b:b + len(r) - c]])
                assert pm.rel_err(got, ref) < TOL[dtype], (round_, len(r))
                a, b = a + c, b + len(r) - c
            for s in slots:
                eng.close(s)
    finally:
        parts.MIXERS.pop("running_mean")


def toy_greedy(tensors, spec, prompt, n, reference=toy_reference):
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(reference(tensors, spec, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out


def test_a_toy_mixer_with_state_generates_through_the_captured_loop(monkeypatch):
    """The same toy model through the Python entry point with the captured decode step: the loop's
    set-up run must leave the sequences' state as it found it, finished rows must not disturb
    the others, and slots that are used again start from zeroed state.  Tokens in float32 are
    those of the whole-sequence reference."""
    from sonicboom_b200 import llm
    from sonicboom_b200.engine.decode import DecodeLoop
    parts.register_mixer("running_mean", RunningMean)
    try:
        spec = toy_spec()
        model = DecoderModel(spec, torch.float32, DEV)
        src = RandomSource(model.tensor_requests(), seed=4, std=0.08, bias_std=0.05, norm_std=0.1)
        tensors = {n: src.tensor(n) for n in src.names()}
        model.bind(lambda n: fetch(src, n, model.dtype, model.device))
        made = []
        real_init = DecodeLoop.__init__

        def spy(self, *a, **k):
            real_init(self, *a, **k)
            made.append(self)
        monkeypatch.setattr(DecodeLoop, "__init__", spy)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (9, 30, 4, 17)]
        budgets = [12, 3, 20, 8]
        eng = sb.Engine(model, max_tokens=64 * 4, n_slots=4)
        from sonicboom_b200.sampling import Sampling
        for round_ in range(2):                    # the second round uses the slots again
            outs = llm.generate_batch(llm.Model(model), prompts, sampling=[Sampling(max_tokens=b) for b in budgets],
                                      ignore_eos=True, engine=eng)
            for p, b, o in zip(prompts, budgets, outs):
                assert o == toy_greedy(tensors, spec, p, b), (round_, len(p))
        assert len(made) >= 2 and all(l.graph is None for l in made)     # captured, then closed
        eng.cache.check()
        assert not eng.cache.records
    finally:
        parts.MIXERS.pop("running_mean")


# -------------------------- a toy architecture with an embedding scale and a logit cap

def test_a_toy_architecture_with_embedding_scale_and_logit_cap(tmp_path):
    """Registered from here, written as a model folder, loaded by name from its config.json and
    generated from: the embedding scale and the logit cap are fields of the model record, so
    nothing in the package changes for an architecture that has them."""
    import json
    from sonicboom_b200 import llm
    from sonicboom_b200.config import ARCHITECTURES, register_architecture

    def to_spec(cfg):
        base = toy_spec(cfg["width"], cfg["vocab"], cfg["layers"])
        layers = tuple(dataclasses.replace(l, mixer=dataclasses.replace(base.layers[0].mixer,
                                                                        prefix=f"toy.layers.{i}.self_attn."))
                       for i, l in enumerate(base.layers))                # attention in every layer
        return dataclasses.replace(base, architecture="ToyCappedForCausalLM", layers=layers,
                                   embedding_scale=float(cfg["embedding_scale"]),
                                   logit_cap=float(cfg["logit_cap"]))

    def reference(tensors, spec, tokens):
        t = dict(tensors)
        t["toy.embed.weight"] = tensors["toy.embed.weight"].float() * spec.embedding_scale
        # the head is the unscaled embedding matrix
        plain = dataclasses.replace(spec, embedding_scale=1.0, logit_cap=0.0)
        x_logits = toy_reference_with_head(t, plain, tokens, tensors["toy.embed.weight"])
        return spec.logit_cap * torch.tanh(x_logits / spec.logit_cap)

    register_architecture("ToyCappedForCausalLM", dict, to_spec)
    try:
        cfg = dict(architectures=["ToyCappedForCausalLM"], width=48, vocab=97, layers=2,
                   embedding_scale=48 ** 0.5, logit_cap=3.0)
        sb.write_random_model(tmp_path, cfg, seed=9, std=0.1, bias_std=0.05, norm_std=0.1)
        assert json.loads((tmp_path / "config.json").read_text())["logit_cap"] == 3.0
        tensors = pm.read_safetensors(tmp_path / "model.safetensors")
        model = llm.model_load(tmp_path, dtype="float32")
        assert model.arch == "ToyCappedForCausalLM"
        spec = model.decoder.spec
        g = torch.Generator().manual_seed(2)
        prompts = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (5, 21)]
        eng = sb.Engine(model.decoder, max_tokens=256)
        for p in prompts:
            s = eng.open()
            got = eng.step([(s, p, list(range(len(p))))]).cpu()
            eng.close(s)
            ref = reference(tensors, spec, p)
            assert float(ref.abs().max()) > 0.5 * spec.logit_cap       # the cap really bends them
            assert pm.rel_err(got, ref) < FP32_TOL
        outs = llm.generate_batch(model, prompts, max_tokens=6, ignore_eos=True)
        for p, o in zip(prompts, outs):
            assert o == toy_greedy(tensors, spec, p, 6, reference)
        with pytest.raises(sb.ConfigError, match="logit_cap"):
            dataclasses.replace(spec, logit_cap=-1.0).validate()
    finally:
        ARCHITECTURES.pop("ToyCappedForCausalLM")


# --------------------------- a toy feed-forward with routing and a toy position encoding

class Top1Experts(parts.FeedForward):
    """Every row goes to the one expert its router score is highest for (float32 scores, the
    lowest index on a tie); an expert is a gated feed-forward of its own.  Experts run on the
    rows routed to them, gathered, through the package's product kernels."""

    def __init__(self, spec, dtype, device):
        self.spec, self.dtype = spec, dtype
        self.n_experts = dict(spec.params)["experts"]
        self.router = self.w_gate_up = self.w_down = None

    def tensor_requests(self):
        p, d, ff = self.spec.prefix, self.spec.width, self.spec.intermediate
        reqs = [TensorRequest(p + "router.weight", (self.n_experts, d))]
        for e in range(self.n_experts):
            reqs += [TensorRequest(f"{p}experts.{e}.gate.weight", (ff, d)),
                     TensorRequest(f"{p}experts.{e}.up.weight", (ff, d)),
                     TensorRequest(f"{p}experts.{e}.down.weight", (d, ff))]
        return reqs

    def bind(self, get):
        from sonicboom_b200.parts.feedforward import interleave_gate_up
        p = self.spec.prefix
        self.router = get(p + "router.weight").float()
        self.w_gate_up = [interleave_gate_up(get(f"{p}experts.{e}.gate.weight"), get(f"{p}experts.{e}.up.weight"))
                          for e in range(self.n_experts)]
        self.w_down = [get(f"{p}experts.{e}.down.weight") for e in range(self.n_experts)]

    def forward(self, h, ctx, residual=None):
        from sonicboom_b200 import ops
        choice = (h.float() @ self.router.t()).argmax(dim=1)
        out = residual if residual is not None else torch.zeros(h.shape[0], self.spec.width, device=h.device)
        for e in range(self.n_experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            x = h[rows].contiguous()
            t = torch.empty(x.shape[0], self.spec.intermediate, dtype=self.dtype, device=h.device)
            ops.linear(x, self.w_gate_up[e], t, ops.EPI_SWIGLU)
            y = torch.zeros(x.shape[0], self.spec.width, device=h.device)
            ops.linear(t, self.w_down[e], y)
            out[rows] += y
        return out


class HalfSpeedRotary(parts.PositionEncoding):
    """Rotates the first half of a head with positions counted at half speed: another table for
    the same rotation kernel."""

    def __init__(self, spec, dtype, device):
        self.head_dim, self.rotary_dim = spec.head_dim, spec.head_dim // 2
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float32)
        self.inv_freq = (0.5 * torch.exp(-2.0 * i / self.rotary_dim * torch.log(torch.tensor(spec.theta)))).to(device)


def half_speed_rope(x, positions, theta):
    """Plain counterpart of HalfSpeedRotary on [n, heads, hd]."""
    hd = x.shape[-1]
    rot = pm.rope_neox(x[..., :hd // 2], positions.float() * 0.5, theta)
    return torch.cat([rot, x[..., hd // 2:]], dim=-1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_routed_feed_forward_and_position_encoding(dtype):
    """A feed-forward that routes rows to experts and a position encoding with its own table,
    both defined here, are registered, built from a spec, given random weights and stepped
    (prompt in two cuts, then single tokens) without a change to the package."""
    parts.register_feed_forward("top1_experts", Top1Experts)
    parts.register_position_encoding("half_speed", HalfSpeedRotary)
    try:
        width, vocab, hd = 64, 101, 32
        layers = []
        for i in range(2):
            p = f"toy.layers.{i}."
            mixer = MixerSpec(kind="attention", width=width, n_heads=2, n_kv_heads=1, head_dim=hd,
                              scale=hd ** -0.5, qkv_bias=False, prefix=p + "self_attn.",
                              position=PositionSpec("half_speed" if i == 0 else "rope_neox", hd, 3000.0))
            ff = (FeedForwardSpec("top1_experts", width, 48, prefix=p + "moe.", params=(("experts", 3),))
                  if i == 0 else FeedForwardSpec("swiglu", width, 80, prefix=p + "mlp."))
            layers.append(LayerSpec("pre_norm", mixer, NormSpec("rmsnorm", width, 1e-6, p + "n1.weight"), ff,
                                    NormSpec("rmsnorm", width, 1e-6, p + "n2.weight")))
        spec = ModelSpec("Toy2", width, vocab, 256, "toy.embed.weight", tuple(layers),
                         (ScheduleEntry(0), ScheduleEntry(1)),
                         NormSpec("rmsnorm", width, 1e-6, "toy.norm.weight"), None)
        model = DecoderModel(spec, DT[dtype], DEV)
        src = RandomSource(model.tensor_requests(), seed=8, std=0.1, norm_std=0.1)
        check(src, model.tensor_requests())
        t = {n: src.tensor(n).float().cpu() for n in src.names()}
        model.bind(lambda n: fetch(src, n, model.dtype, model.device))

        def reference(tokens):
            n = len(tokens)
            pos = torch.arange(n)
            x = pm.embedding(t["toy.embed.weight"], tokens)
            for i in range(2):
                p = f"toy.layers.{i}."
                h = pm.rms_norm(x, t[p + "n1.weight"], 1e-6)
                a = p + "self_attn."
                q = pm.linear(h, t[a + "q_proj.weight"]).view(n, 2, hd)
                k = pm.linear(h, t[a + "k_proj.weight"]).view(n, 1, hd)
                v = pm.linear(h, t[a + "v_proj.weight"]).view(n, 1, hd)
                if i == 0:
                    q, k = half_speed_rope(q, pos, 3000.0), half_speed_rope(k, pos, 3000.0)
                else:
                    q, k = pm.rope_neox(q, pos, 3000.0), pm.rope_neox(k, pos, 3000.0)
                x = x + pm.linear(pm.attention(q, k, v, pos, pos, hd ** -0.5).reshape(n, 2 * hd), t[a + "o_proj.weight"])
                f = pm.rms_norm(x, t[p + "n2.weight"], 1e-6)
                if i == 0:
                    m = p + "moe."
                    choice = (f @ t[m + "router.weight"].t()).argmax(dim=1)
                    y = torch.zeros_like(x)
                    for e in range(3):
                        rows = choice == e
                        y[rows] = pm.swiglu_mlp(f[rows], t[f"{m}experts.{e}.gate.weight"],
                                                t[f"{m}experts.{e}.up.weight"], t[f"{m}experts.{e}.down.weight"])
                    x = x + y
                else:
                    x = x + pm.swiglu_mlp(f, t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"],
                                          t[p + "mlp.down_proj.weight"])
            return pm.linear(pm.rms_norm(x, t["toy.norm.weight"], 1e-6), t["toy.embed.weight"]), None

        eng = sb.Engine(model, max_tokens=512)
        g = torch.Generator().manual_seed(3)
        reqs = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (70, 9)]
        slots = [eng.open() for _ in reqs]
        cuts = [40, 5]
        got = [[], []]
        out = eng.step([(s, r[:c], list(range(c))) for s, r, c in zip(slots, reqs, cuts)]).cpu()
        got[0].append(out[:cuts[0]]); got[1].append(out[cuts[0]:])
        out = eng.step([(s, r[c:c + 2], [0, 1]) for s, r, c in zip(slots, reqs, cuts)]).cpu()
        got[0].append(out[:2]); got[1].append(out[2:])
        for step in range(2, 4):                    # then a token each
            out = eng.step([(s, [r[c + step]], [0]) for s, r, c in zip(slots, reqs, cuts)]).cpu()
            got[0].append(out[:1]); got[1].append(out[1:])
        for r, c, pieces in zip(reqs, cuts, got):
            ref, _ = reference(r[:c + 4])
            # a row whose two best router scores nearly tie may go to the other expert in bfloat16
            err = (torch.cat(pieces) - ref).abs().amax(dim=1) / ref.abs().max()
            assert float(err.median()) < TOL[dtype] and float((err < TOL[dtype]).float().mean()) > 0.9, err
            if dtype == "float32":
                assert float(err.max()) < TOL[dtype]
    finally:
        parts.FEED_FORWARDS.pop("top1_experts")
        parts.POSITION_ENCODINGS.pop("half_speed")


def test_unknown_kinds_are_refused():
    spec = toy_spec()
    with pytest.raises(sb.ConfigError, match="running_mean"):
        DecoderModel(spec, torch.float32, DEV)
