"""The Python entry point, in the manner of the reference's `boom_llm_*` C ABI and its Guile
binding (capi/include/sonicboom/capi.h:600-783, bindings/guile/scheme/sonicboom/
inference.scm:186,266,586-620): load a model, make a session with a context length, prefill
token ids, decode with a sampling record and a per-token callback; `generate` does all of it.
Token ids go in and come out (the reference's tokenizer belongs to its GGUF files and is not
part of this library).  Beyond the reference, `generate_batch` runs many prompts as batches.
"""
from __future__ import annotations

from typing import Callable, Optional

from .engine import Engine
from .engine.generate import generate as _generate
from .models import load_model, random_model
from .sampling import Sampler, Sampling


class Model:
    """A loaded model (`boom_llm_model`)."""

    def __init__(self, decoder):
        self.decoder = decoder

    @property
    def arch(self) -> str:
        """The architecture name the model's configuration declares (`boom_llm_model_arch`)."""
        return self.decoder.spec.architecture

    @property
    def eos(self) -> tuple:
        """The model's end-of-sequence token ids (`boom_llm_model_eos`); may be empty."""
        return tuple(self.decoder.spec.stop_tokens)

    @property
    def vocab_size(self) -> int:
        return self.decoder.spec.vocab


def model_load(path, dtype: str = "bfloat16", device: str = "cuda:0") -> Model:
    """`boom_llm_model_load`: a model folder (config.json + safetensors) to a model on the
    device.  `dtype` "bfloat16" serves; "float32" runs everything in true 32-bit."""
    return Model(load_model(path, dtype=dtype, device=device))


def model_random(config: dict, seed: int, dtype: str = "bfloat16", device: str = "cuda:0",
                 **init) -> Model:
    """A model with seeded random weights, made on the device from a config.json dictionary."""
    return Model(random_model(config, seed, dtype=dtype, device=device, **init))


class Session:
    """One conversation's tokens and cache (`boom_llm_session`): prefill, then decode.

    Decode continues from where the previous call stopped, so `max_tokens=1` calls are
    per-token steps; the sampled draw is keyed by absolute position, so the same seed gives the
    same tokens however the calls are cut."""

    def __init__(self, model: Model, n_ctx: int):
        if n_ctx <= 0:
            raise ValueError("n_ctx must be > 0")
        self.model = model
        self.n_ctx = min(int(n_ctx), model.decoder.spec.max_positions)
        self.engine = Engine(model.decoder, max_tokens=self.n_ctx, n_slots=1)
        self.sampler = Sampler(model.decoder.device)
        self.slot = None
        self.tokens: list = []          # prompt + everything decoded so far
        self._logits = None             # logits at the last position, for the next token
        self._pending = None            # a produced token that was not fed to the model yet
        self._loop = None               # the captured decode step while one is open
        self._loop_key = None           # the sampling fields that loop was captured with

    def _close_loop(self) -> None:
        loop, self._loop, self._loop_key = self._loop, None, None
        if loop is not None:
            loop.close()

    def _loop_for(self, s: Sampling):
        """The captured decode step for this sampling record (made at the first token that
        needs it and kept until the prompt, the record or the context's end changes that), or
        None when the engine cannot capture it (penalties read the token history on the host)."""
        key = (s.temperature, s.top_p, s.top_k, s.seed, s.min_p)
        if self._loop is not None and self._loop_key != key:
            self._close_loop()
        if self._loop is None:
            room = self.n_ctx - self.engine.length(self.slot)
            self._loop = self.engine.decode_loop([self.slot], [room], [s])
            self._loop_key = key if self._loop is not None else None
        return self._loop

    def prefill(self, tokens) -> int:
        """`boom_llm_prefill`: sets the prompt.  Returns how many leading tokens were reused
        from the cache of the previous prompt; the last prompt token is always processed."""
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise ValueError("prefill needs a non-empty prompt")
        if len(tokens) > self.n_ctx:
            raise ValueError(f"prompt of {len(tokens)} tokens exceeds n_ctx = {self.n_ctx}")
        self._close_loop()
        reused = 0
        if self.slot is not None:
            common = 0
            for a, b in zip(self.tokens[:self.engine.length(self.slot)], tokens):
                if a != b:
                    break
                common += 1
            reused = min(common, len(tokens) - 1)
            if not self.engine.cache.truncate(self.slot, reused):
                reused = 0
        if self.slot is not None and reused == 0:
            self.engine.close(self.slot)
            self.slot = None
        if self.slot is None:
            self.slot = self.engine.open()
        rest = tokens[reused:]
        self._logits = self.engine.step([(self.slot, rest, [len(rest) - 1])])
        self._pending = None
        self.tokens = tokens
        return reused

    def decode(self, sampling: Sampling, cb: Optional[Callable] = None) -> list:
        """`boom_llm_decode`: up to sampling.max_tokens tokens; `cb(token)` is called for each
        in order and a non-zero return stops the decode.  Returns the tokens produced.  The
        first token after a prefill comes from the prefill's logits; every later one from the
        captured decode step (one graph launch per token, the token id in and out through pinned
        host memory), as the reference replays its captured step per token
        (core/src/model/gemma4_plan.cpp:1650-1696)."""
        if self.slot is None or (self._logits is None and self._pending is None):
            raise RuntimeError("decode requires a prompt: call prefill first")
        s = sampling.checked()
        out = []
        while len(out) < s.max_tokens:
            if len(self.tokens) >= self.n_ctx:
                raise RuntimeError(f"the session's context of {self.n_ctx} tokens is full")
            if self._logits is not None:
                (tok,) = self.sampler.sample(self._logits, [s], [len(self.tokens)], [self.tokens])
                self._logits = None
            else:                                # feed the last token, get the next
                loop = self._loop_for(s)
                if loop is not None:
                    (tok,) = loop.step_host([self._pending])
                else:
                    logits = self.engine.step([(self.slot, [self._pending], [0])])
                    (tok,) = self.sampler.sample(logits, [s], [len(self.tokens)], [self.tokens])
            out.append(tok)
            self.tokens.append(tok)
            self._pending = tok
            if cb is not None and cb(tok):
                break
        return out

    def free(self) -> None:
        self._close_loop()
        if self.slot is not None:
            self.engine.close(self.slot)
            self.slot = None


def session_new(model: Model, n_ctx: int) -> Session:
    """`boom_llm_session_new`."""
    return Session(model, n_ctx)


def generate_tokens(session: Session, prompt, max_tokens: int, prefill: bool = True, *,
                    temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                    min_p: float = 0.0, seed: int = 0, repeat_penalty: float = 1.0,
                    repeat_last_n: int = 64, presence_penalty: float = 0.0,
                    frequency_penalty: float = 0.0, cb: Optional[Callable] = None) -> list:
    """The binding's `generate-tokens` (inference.scm:545-585): prefill the prompt's token
    ids, decode up to `max_tokens`, return the produced ids.  Temperature 0 is greedy."""
    if prefill:
        session.prefill(prompt)
    return session.decode(Sampling(temperature=temperature, top_p=top_p, top_k=top_k, seed=seed,
                                   max_tokens=max_tokens, min_p=min_p,
                                   repeat_penalty=repeat_penalty, repeat_last_n=repeat_last_n,
                                   presence_penalty=presence_penalty,
                                   frequency_penalty=frequency_penalty), cb)


def generate_batch(model: Model, prompts: list, max_tokens: int = 16, *, sampling=None,
                   stop_tokens=None, ignore_eos: bool = False, on_token=None,
                   max_cache_tokens: Optional[int] = None, max_batch: Optional[int] = None,
                   engine: Optional[Engine] = None, **sampling_fields) -> list:
    """Generates for many prompts (lists of token ids) at once.

    `sampling` is a Sampling (or one per prompt); without it one is made from `max_tokens`
    and the keyword fields (temperature, top_k, top_p, min_p, seed, repeat_penalty,
    repeat_last_n, presence_penalty, frequency_penalty).  Stop tokens default to the model's
    end-of-sequence ids unless `ignore_eos`.  The prompts run as one batch when the cache
    holds them, else as several batches one after another."""
    if sampling is None:
        sampling = Sampling(max_tokens=max_tokens, **sampling_fields)
    if stop_tokens is None:
        stop_tokens = () if ignore_eos else model.eos
    if engine is None:
        page = 64
        need = sum((len(p) + (sampling.max_tokens if isinstance(sampling, Sampling)
                              else max(s.max_tokens for s in sampling)) + page - 1) // page * page
                   for p in prompts)
        engine = Engine(model.decoder, max_tokens=min(need, max_cache_tokens or need))
    return _generate(engine, Sampler(model.decoder.device), prompts, sampling, stop_tokens,
                     on_token, max_batch, model.decoder.spec.max_positions)
