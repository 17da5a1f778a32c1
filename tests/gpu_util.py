"""Helpers shared by the GPU tests: loaded engines, and replaying requests in several cuts."""
import functools

import torch

import plain_model as pm
import sonicboom_b200 as sb


@functools.lru_cache(maxsize=None)
def _load(model_dir: str, dtype: str):
    return sb.load_model(model_dir, dtype=dtype)


def engine_for(model_dirs, name, dtype, max_tokens=4096):
    return sb.Engine(_load(str(model_dirs[name]), dtype), max_tokens=max_tokens)


def whole(engine, tokens):
    """Logits at every position of one request, alone, in one step."""
    s = engine.open()
    out = engine.step([(s, tokens, list(range(len(tokens))))]).float().cpu()
    engine.close(s)
    return out


def tail_one_by_one(engine, tokens, n_tail=32):
    """The same request with its last n_tail tokens fed one by one."""
    s = engine.open()
    k = len(tokens) - n_tail
    outs = [engine.step([(s, tokens[:k], list(range(k)))]).float().cpu()]
    for t in tokens[k:]:
        outs.append(engine.step([(s, [t], [0])]).float().cpu())
    engine.close(s)
    return torch.cat(outs)


def batch_unequal(engine, requests, prompt_lens):
    """Requests that start together: request i brings its first prompt_lens[i] tokens in the
    first step and then one token a step; a request whose tokens are used up ends (its slot
    is closed) while the others go on.  Returns each request's logits at every position."""
    slots = [engine.open() for _ in requests]
    outs = [[] for _ in requests]
    lg = engine.step([(s, r[:k], list(range(k))) for s, r, k in zip(slots, requests, prompt_lens)])
    at = 0
    for i, k in enumerate(prompt_lens):
        outs[i].append(lg[at:at + k].float().cpu())
        at += k
    fed = list(prompt_lens)
    live = [i for i, r in enumerate(requests) if fed[i] < len(r)]
    for i in set(range(len(requests))) - set(live):
        engine.close(slots[i])
    while live:
        lg = engine.step([(slots[i], [requests[i][fed[i]]], [0]) for i in live]).float().cpu()
        for row, i in enumerate(live):
            outs[i].append(lg[row:row + 1])
            fed[i] += 1
        for i in [i for i in live if fed[i] == len(requests[i])]:
            engine.close(slots[i])
        live = [i for i in live if fed[i] < len(requests[i])]
    return [torch.cat(o) for o in outs]


def oracle_logits(oracles, name, tokens, schedule=None):
    cfg, tensors = oracles[name]
    return pm.forward(cfg, tensors, tokens, schedule=schedule)
