"""A decode session: a fixed set of live requests, one token each per step.

This is the inner loop of generation once prompts are in the cache.  It runs the engine's own
step function; what it adds is that the step's shape does not change from one step to the next,
so the work of a step can be recorded once and replayed.
"""
from __future__ import annotations

from typing import Hashable, List, Sequence

import torch

from .engine import Engine, StepEntry


class DecodeSession:
    def __init__(self, engine: Engine, request_ids: Sequence[Hashable]):
        self.engine = engine
        self.request_ids = list(request_ids)
        self.h2d_bytes_per_step = 0

    def step(self, tokens: Sequence[int]) -> torch.Tensor:
        """Feed one token per request (in the session's order); float32 logits [requests, vocab] on the device."""
        entries = [StepEntry(rid, [int(t)], [0]) for rid, t in zip(self.request_ids, tokens)]
        logits = self.engine.step(entries)
        self.h2d_bytes_per_step = self.engine.last_h2d_bytes
        return logits

    def close(self) -> None:
        pass
