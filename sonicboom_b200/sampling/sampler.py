"""Runs the device sampler for the rows of one step.

One kernel launch picks a token for every row: the greedy argmax or the reference's seeded
sampler (penalties, 256 candidates, 30-logit window, top-k, min-p, nucleus, Gumbel-max with
Philox keyed by seed, absolute position and token id; core/src/nn/sampling.cpp:157-352).  The
draw's key holds the position of the token being produced, never the row, so a sequence's
tokens do not depend on the batch it runs in."""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .params import Sampling

_RECORD = np.dtype([("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"),
                    ("repeat_penalty", "<f4"), ("presence_penalty", "<f4"),
                    ("frequency_penalty", "<f4"), ("top_k", "<u4"), ("history_len", "<i4"),
                    ("seed", "<u8"), ("position", "<u8")])


def pack_params(samplings: list[Sampling], positions: list[int], histories: list) -> tuple:
    """(records as a uint8 array, history int32 array or None) for the kernel."""
    n = len(samplings)
    rec = np.zeros(n, dtype=_RECORD)
    windows = []
    for i, (s, pos, hist) in enumerate(zip(samplings, positions, histories)):
        win = list(hist[-s.repeat_last_n:]) if s.penalizes and s.repeat_last_n > 0 else []
        windows.append(win)
        rec[i] = (s.temperature, s.top_p, s.min_p, s.repeat_penalty, s.presence_penalty,
                  s.frequency_penalty, s.top_k, len(win), s.seed, pos)
    stride = max((len(w) for w in windows), default=0)
    history = None
    if stride > 0:
        history = np.full((n, stride), -1, dtype=np.int32)
        for i, w in enumerate(windows):
            history[i, :len(w)] = w
    return rec.view(np.uint8).reshape(-1), history


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        if _RECORD.itemsize != ops.sample_params_size():
            raise RuntimeError("sampler record layout differs between Python and the kernel library")

    def sample(self, logits: torch.Tensor, samplings: list[Sampling], positions: list[int],
               histories: list) -> list[int]:
        """One token for every row of `logits`; `positions[i]` is the absolute position of
        the token row i produces, `histories[i]` that sequence's tokens so far."""
        rec, history = pack_params(samplings, positions, histories)
        params = torch.from_numpy(rec).to(self.device)
        hist = torch.from_numpy(history).to(self.device) if history is not None else None
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        ops.sample(logits, params, hist, out)
        ids = out.cpu().tolist()
        ops.check_status()           # the host has just waited for the step: a cheap place to look
        return ops.check_tokens(ids)
