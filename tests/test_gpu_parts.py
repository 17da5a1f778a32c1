"""Each part alone against the plain implementation, the run order as data (a layer twice, a
layer reading another's cache), and a toy mixer with state of its own that is registered,
built and stepped without a change to the package."""
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


def toy_reference(tensors, spec, tokens):
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
    return pm.linear(pm.rms_norm(x, t["toy.norm.weight"], 1e-5), t["toy.embed.weight"])


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


def test_unknown_kinds_are_refused():
    spec = toy_spec()
    with pytest.raises(sb.ConfigError, match="running_mean"):
        DecoderModel(spec, torch.float32, DEV)
