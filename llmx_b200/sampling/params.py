"""Sampling settings: names, defaults and ranges as the reference's `infer::Sampling`
(src/inference/sampler.hpp:43-65; the command line's flags src/cli/main.cpp:2018-2031)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple


@dataclass(frozen=True)
class SamplingParams:
    max_tokens: int = 64            # -n / --max-tokens: tokens generated at most
    temp: float = 0.8               # --temp: 0 is greedy
    top_k: int = 40                 # --topk: 0 keeps every token
    top_p: float = 0.95             # --topp: 1 keeps every token
    min_p: float = 0.0              # --min-p
    penalty: float = 1.0            # --penalty: repetition penalty, 1 is none
    presence_penalty: float = 0.0   # --presence-penalty
    frequency_penalty: float = 0.0  # --frequency-penalty
    seed: int = 0                   # --seed: 0 keeps the generator's fixed default state
    ignore_eos: bool = False        # --ignore-eos: the token that ends a reply is never drawn
    stop_token_ids: Tuple[int, ...] = ()   # extra ids that end a reply (beside the model's eos)

    def __post_init__(self) -> None:
        def finite(v):
            return isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(v)
        if not isinstance(self.max_tokens, int) or self.max_tokens < 1:
            raise ValueError("max_tokens must be an integer of at least 1")
        if not finite(self.temp) or self.temp < 0:
            raise ValueError("temp must be a finite number of at least 0")
        if not isinstance(self.top_k, int) or self.top_k < 0:
            raise ValueError("top_k must be an integer of at least 0")
        if not finite(self.top_p) or not 0.0 <= self.top_p <= 1.0:
            raise ValueError("top_p must lie in 0..1")
        if not finite(self.min_p) or not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must lie in 0..1")
        if not finite(self.penalty) or self.penalty < 1.0:
            raise ValueError("penalty must be at least 1")
        for name in ("presence_penalty", "frequency_penalty"):
            v = getattr(self, name)
            if not finite(v) or not -2.0 <= v <= 2.0:
                raise ValueError(f"{name} must lie in -2..2")
        if not isinstance(self.seed, int) or not 0 <= self.seed < 2 ** 64:
            raise ValueError("seed must be an unsigned 64-bit integer")

    @property
    def greedy(self) -> bool:
        return self.temp <= 0.0

    @property
    def penalized(self) -> bool:
        return (self.penalty > 0 and self.penalty != 1.0) or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0


GREEDY = SamplingParams(temp=0.0, top_k=0, top_p=1.0)
