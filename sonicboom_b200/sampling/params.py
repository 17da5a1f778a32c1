"""Sampling parameters, with the names, defaults and meanings of the reference's
`boom_llm_sampling` (capi/include/sonicboom/capi.h:629-677): zero means "off" throughout,
temperature 0 is greedy, and a range error names the field (capi/src/capi.cpp:2610-2660)."""
from __future__ import annotations

import math
from dataclasses import dataclass

MAX_PENALTY_WINDOW = 1024      # the device penalty window's cap (capi/src/capi.cpp:2711-2715)


@dataclass(frozen=True)
class Sampling:
    temperature: float = 0.0       # 0: greedy argmax, ties toward the lowest id
    top_p: float = 1.0             # 1 (or 0): no nucleus truncation
    top_k: int = 0                 # 0: no top-k truncation
    seed: int = 0
    max_tokens: int = 16
    min_p: float = 0.0             # 0: keep every candidate above the logit window
    repeat_penalty: float = 1.0    # 1 (or 0): no repetition penalty
    repeat_last_n: int = 64        # penalty window in tokens; 0 disables every penalty
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0

    def checked(self) -> "Sampling":
        """Validated copy with the neutral forms filled in; errors name the field."""
        def bad(name, why):
            raise ValueError(f"sampling.{name}: {why}")
        for name in ("temperature", "top_p", "min_p", "repeat_penalty", "presence_penalty",
                     "frequency_penalty"):
            v = getattr(self, name)
            if isinstance(v, bool) or not isinstance(v, (int, float)) or math.isnan(v) or math.isinf(v):
                bad(name, f"must be a finite number, got {v!r}")
        for name in ("top_k", "seed", "max_tokens", "repeat_last_n"):
            v = getattr(self, name)
            if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                bad(name, f"must be a non-negative integer, got {v!r}")
        if self.temperature < 0:
            bad("temperature", "must be >= 0")
        if not 0.0 <= self.top_p <= 1.0:
            bad("top_p", "must be in [0, 1]")
        if not 0.0 <= self.min_p <= 1.0:
            bad("min_p", "must be in [0, 1]")
        if self.repeat_penalty < 0:
            bad("repeat_penalty", "must be >= 0 (0 and 1 both mean off)")
        if self.repeat_last_n > MAX_PENALTY_WINDOW:
            bad("repeat_last_n", f"above the device penalty window's cap of {MAX_PENALTY_WINDOW}")
        if self.seed >= 2 ** 64:
            bad("seed", "must fit 64 bits")
        rp = 1.0 if self.repeat_penalty == 0 else float(self.repeat_penalty)
        return Sampling(float(self.temperature), float(self.top_p), int(self.top_k), int(self.seed),
                        int(self.max_tokens), float(self.min_p), rp, int(self.repeat_last_n),
                        float(self.presence_penalty), float(self.frequency_penalty))

    @property
    def penalizes(self) -> bool:
        return self.repeat_last_n > 0 and (self.repeat_penalty != 1.0 or self.presence_penalty != 0.0
                                           or self.frequency_penalty != 0.0)
