"""Plain implementation of token sampling as hardenedlinux/SonicBoom defines it, used only
as the test oracle.  Pure Python/numpy, one function per stage, written from
core/src/nn/sampling.cpp and core/include/sonicboom/nn/sampling.h (cited per function).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

SAMPLE_CANDIDATES = 256        # core/include/sonicboom/nn/sampling.h:68  (kSampleCandidates)
SAMPLE_LOGIT_WINDOW = 30.0     # core/include/sonicboom/nn/sampling.h:61  (kSampleLogitWindow)


@dataclass
class Params:
    """Neutral defaults of core/include/sonicboom/nn/sampling.h:47-57."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 0
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0


def philox4x32_10(counter, key: int):
    """Philox4x32-10 with the Random123 constants and a 64-bit key
    (core/src/nn/sampling.cpp:207-227).  Known answer: counter 0, key 0 ->
    6627e8d5 e169c58d bc57ac4c 9b00dbd8."""
    m0, m1, w0, w1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c0, c1, c2, c3 = [int(c) & 0xFFFFFFFF for c in counter]
    k0, k1 = key & 0xFFFFFFFF, (key >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0 = m0 * c0
        p1 = m1 * c2
        hi0, lo0 = p0 >> 32, p0 & 0xFFFFFFFF
        hi1, lo1 = p1 >> 32, p1 & 0xFFFFFFFF
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0 = (k0 + w0) & 0xFFFFFFFF
        k1 = (k1 + w1) & 0xFFFFFFFF
    return [c0, c1, c2, c3]


def apply_penalties(logits: np.ndarray, p: Params, history) -> np.ndarray:
    """Over the last repeat_last_n history tokens, for a token seen c times:
    v = v/rp if v > 0 else v*rp (when rp != 1), then v -= freq*c + presence, each a
    single float32 operation (core/src/nn/sampling.cpp:77-105)."""
    adv = logits.astype(np.float32).copy()
    if len(history) == 0 or (p.repeat_penalty == 1.0 and p.presence_penalty == 0.0
                             and p.frequency_penalty == 0.0):
        return adv
    window = min(len(history), int(p.repeat_last_n))
    count: dict[int, int] = {}
    for t in history[len(history) - window:]:
        if 0 <= t < len(adv):
            count[t] = count.get(t, 0) + 1
    rp = np.float32(p.repeat_penalty)
    for t, c in count.items():
        v = adv[t]
        if p.repeat_penalty != 1.0:
            v = np.float32(v / rp) if v > 0 else np.float32(v * rp)
        adjust = np.float32(np.float32(p.frequency_penalty) * np.float32(c)
                            + np.float32(p.presence_penalty))
        adv[t] = np.float32(v - adjust)
    return adv


def argmax(x: np.ndarray) -> int:
    """First maximum: ties go to the lowest id (core/src/nn/sampling.cpp:238-244)."""
    best = 0
    for i in range(1, len(x)):
        if x[i] > x[best]:
            best = i
    return best


def select_candidates(logits: np.ndarray, p: Params, history):
    """z = penalized logit / T as one float32 division; the 256 highest z survive in
    (z descending, id ascending) order (core/src/nn/sampling.cpp:257-285)."""
    adv = apply_penalties(logits, p, history)
    z = (adv / np.float32(p.temperature)).astype(np.float32)
    order = sorted(range(len(z)), key=lambda i: (-float(z[i]), i))
    return [(i, float(z[i])) for i in order[:SAMPLE_CANDIDATES]]


def filter_candidates(cands, p: Params):
    """Logit window of 30 below the maximum, top-k, min-p (z < max + ln(min_p) dropped),
    nucleus: the shortest descending prefix whose normalized mass reaches top_p
    (core/src/nn/sampling.cpp:157-203)."""
    if not cands:
        return []
    m = cands[0][1]
    floor_z = np.float32(np.float32(m) - np.float32(SAMPLE_LOGIT_WINDOW))
    out = [c for c in cands if np.float32(c[1]) >= floor_z]
    if p.top_k > 0 and len(out) > p.top_k:
        out = out[:p.top_k]
    if p.min_p > 0.0:
        cutoff = np.float32(np.float32(m) + np.float32(math.log(np.float32(p.min_p))))
        out = [c for c in out if np.float32(c[1]) >= cutoff]
    if 0.0 < p.top_p < 1.0 and out:
        total = sum(math.exp(c[1] - m) for c in out)
        if total > 0.0:
            acc, keep = 0.0, 0
            while keep < len(out):
                acc += math.exp(out[keep][1] - m)
                keep += 1
                if acc / total >= float(np.float32(p.top_p)):
                    break
            out = out[:max(keep, 1)]
    return out


def draw(kept, p: Params, position: int) -> int:
    """Gumbel-max: u = (bits[0]+0.5)/2^32 with bits = philox({pos_lo, pos_hi, id, 0}, seed),
    g = -log(-log u), the highest z+g wins, ties toward the lower id
    (core/src/nn/sampling.cpp:287-312)."""
    best, best_score = -1, -math.inf
    for tok, z in kept:
        bits = philox4x32_10([position & 0xFFFFFFFF, position >> 32, tok, 0], p.seed)
        u = (bits[0] + 0.5) / 4294967296.0
        score = z + (-math.log(-math.log(u)))
        if best < 0 or score > best_score or (score == best_score and tok < best):
            best, best_score = tok, score
    return best


def sample_token(logits: np.ndarray, p: Params, position: int, history=()) -> int:
    """Penalties, then the argmax for temperature <= 0, else candidates, filters and the
    draw; `position` is the absolute position of the token being produced
    (core/src/nn/sampling.cpp:314-352)."""
    if not p.temperature > 0.0:
        return argmax(apply_penalties(logits, p, list(history)))
    cands = select_candidates(logits, p, list(history))
    return draw(filter_candidates(cands, p), p, position)
