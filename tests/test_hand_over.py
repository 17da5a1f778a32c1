"""The hand-over of a norm (and of an L2 hint) from the part that runs to the one that follows:
the decisions of `StepContext.linear` / `take_normed`, with the product itself replaced by a
recorder.  No GPU is needed."""
import torch

from sonicboom_b200 import ops
from sonicboom_b200.parts.base import Norm, StepContext


class RmsLike(Norm):
    def __init__(self, width):
        self.w, self.eps = torch.ones(width), 1e-5

    def as_rms(self):
        return self.w, self.eps


class OtherNorm(Norm):          # a norm that is no RMS norm: offers nothing to a product kernel
    pass


def recorder(monkeypatch):
    calls = []

    def linear(a, w, out, epilogue=ops.EPI_NONE, bias=None, residual=None, kernel="auto", norm=None,
               warm=None):
        calls.append(dict(epilogue=epilogue, norm=norm, warm=warm))
        if norm is not None:
            norm[2].fill_(7.0)
        return out
    monkeypatch.setattr(ops, "linear", linear)
    return calls


def operands(rows=3, k=8, n=4):
    return torch.zeros(rows, k, dtype=torch.bfloat16), torch.zeros(n, k, dtype=torch.bfloat16), \
        torch.zeros(rows, n)


def test_a_named_rms_norm_rides_on_the_product_and_is_taken_once(monkeypatch):
    calls = recorder(monkeypatch)
    ctx = StepContext(plan=None, cache=None)
    a, w, out = operands()
    norm = RmsLike(4)
    ctx.next_norm = norm
    assert ctx.linear(a, w, out, ops.EPI_RESIDUAL, residual=out) is out
    weight, eps, normed = calls[0]["norm"]
    assert weight is norm.w and eps == norm.eps
    assert normed.dtype == torch.bfloat16 and normed.shape == out.shape      # the activation dtype
    assert ctx.next_norm is None                                             # a request is used once
    got = ctx.take_normed(norm, out)
    assert got is normed and float(got[0, 0]) == 7.0
    assert ctx.take_normed(norm, out) is None                                # and handed over once


def test_nothing_is_handed_to_the_wrong_norm_or_for_other_rows(monkeypatch):
    recorder(monkeypatch)
    a, w, out = operands()
    norm = RmsLike(4)
    ctx = StepContext(plan=None, cache=None)
    ctx.next_norm = norm
    ctx.linear(a, w, out, ops.EPI_NONE)
    assert ctx.take_normed(RmsLike(4), out) is None          # another norm object
    ctx.next_norm = norm
    ctx.linear(a, w, out, ops.EPI_NONE)
    assert ctx.take_normed(norm, out.clone()) is None        # not the rows that were normed
    ctx.next_norm = norm
    ctx.linear(a, w, out, ops.EPI_NONE)
    ctx.linear(a, w, out, ops.EPI_NONE)                      # a later product without a request
    assert ctx.take_normed(norm, out) is None                # forgets the earlier one


def test_no_request_no_norm(monkeypatch):
    calls = recorder(monkeypatch)
    a, w, out = operands()
    ctx = StepContext(plan=None, cache=None)
    ctx.linear(a, w, out, ops.EPI_NONE)                      # nobody named a norm
    ctx.next_norm = OtherNorm()
    ctx.linear(a, w, out, ops.EPI_NONE)                      # a norm that is not an RMS norm
    ctx.next_norm = RmsLike(4)
    ctx.linear(a, w, torch.zeros(3, 2, dtype=torch.bfloat16), ops.EPI_SWIGLU)   # no float32 rows to norm
    assert [c["norm"] for c in calls] == [None, None, None]
    assert ctx.take_normed(RmsLike(4), out) is None


def test_an_l2_hint_goes_with_the_next_product_only(monkeypatch):
    calls = recorder(monkeypatch)
    a, w, out = operands()
    ctx = StepContext(plan=None, cache=None)
    hint = torch.zeros(16)
    ctx.next_weights = hint
    ctx.linear(a, w, out, ops.EPI_NONE)
    ctx.linear(a, w, out, ops.EPI_NONE)
    assert calls[0]["warm"] is hint and calls[1]["warm"] is None


# ------------------------------------------------------------------ the block's use of it
def build_block(monkeypatch, mixer_hands_over: bool):
    """A pre-norm block out of toy parts registered for this test: norms that count their own
    runs, a mixer and a feed-forward that add 1 to the residual; the mixer leaves the next norm's
    result behind (as a product kernel would) only if asked to."""
    from sonicboom_b200 import parts
    from sonicboom_b200.config.specs import FeedForwardSpec, LayerSpec, MixerSpec, NormSpec
    from sonicboom_b200.parts.base import BLOCKS, FeedForward, Mixer

    runs = []

    class CountingNorm(RmsLike):
        def __init__(self, spec, dtype, device):
            super().__init__(spec.width)
            self.name = spec.tensor

        def forward(self, x, out_dtype, rows=None):
            runs.append(self.name)
            return x.to(out_dtype)

    class AddOne(Mixer):
        def __init__(self, spec, dtype, device):
            pass

        def forward(self, h, ctx, residual=None):
            out = residual.add_(1.0)
            if mixer_hands_over and ctx.next_norm is not None:
                ctx._normed = (ctx.next_norm, out, out.to(torch.bfloat16))
            return out

    class AddOneFF(FeedForward):
        def __init__(self, spec, dtype, device):
            pass

        def forward(self, h, ctx, residual=None):
            assert ctx.next_norm is ctx.after_block_norm       # what follows the block follows it
            return residual.add_(1.0)

    monkeypatch.setitem(parts.base.NORMS, "counting", CountingNorm)
    monkeypatch.setitem(parts.base.MIXERS, "add_one", AddOne)
    monkeypatch.setitem(parts.base.FEED_FORWARDS, "add_one", AddOneFF)
    spec = LayerSpec(arrangement="pre_norm", mixer=MixerSpec(kind="add_one", width=4),
                     mixer_norm=NormSpec("counting", 4, 1e-5, "first"),
                     feed_forward=FeedForwardSpec(kind="add_one", width=4, intermediate=8),
                     feed_forward_norm=NormSpec("counting", 4, 1e-5, "second"))
    return BLOCKS["pre_norm"](spec, torch.bfloat16, "cpu"), runs


def test_a_block_runs_the_norms_itself_when_nothing_is_handed_over(monkeypatch):
    block, runs = build_block(monkeypatch, mixer_hands_over=False)
    ctx = StepContext(plan=None, cache=None)
    x = torch.zeros(2, 4)
    assert float(block.forward(x, ctx)[0, 0]) == 2.0
    assert runs == ["first", "second"]
    assert block.input_norm() is block.mixer_norm


def test_a_block_takes_what_is_handed_over(monkeypatch):
    block, runs = build_block(monkeypatch, mixer_hands_over=True)
    ctx = StepContext(plan=None, cache=None)
    x = torch.zeros(2, 4)
    ctx._normed = (block.mixer_norm, x, x.to(torch.bfloat16))   # left by the entry before it
    ctx.after_block_norm = RmsLike(4)
    block.forward(x, ctx)
    assert runs == []                                           # neither norm ran as its own kernel
