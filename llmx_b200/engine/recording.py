"""Recorded steps: a step's shape recorded once as a CUDA graph and replayed.

The kernels a step launches, their grids and the buffers they use depend on how many rows each request
brings, on which rows' logits are wanted and on how much context the block tables have room for -- not on the
requests' histories, tokens or pages, which the kernels read from the step's metadata on the device.  A
`Recording` holds the CUDA graph of one such shape and the static metadata buffer it reads; a step of the same
shape then costs one host-to-device copy and one graph launch.  What is recorded is the model's own forward
pass over the engine's own cache.

What the model's parts decide on the host from a shape (their launch plans, parts/base.py) is decided once,
for the recording's room, when the recording is made; every run only refills the plans' ints.  This module
knows no part's plan.

The engine makes a recording of a shape once it has seen it `EngineOptions.record_after` times
(`Engine.step(..., record=True)`): a scheduler that cuts long prompts into portions of its token budget brings
the same shape step after step.  Decode sessions (decode_loop.py) record the shape "one row for each of b
requests" the same way.
"""
from __future__ import annotations

import gc
from typing import Callable, Optional, Sequence

import numpy as np
import torch

from ..parts.base import StepShape
from .batch import StepLayout

MAX_STEP_RECORDINGS = 16   # recordings of general shapes an engine keeps (least recently used goes first)


class _NoCache:
    """Stands in for a request's cache while the static views are made (only the state slots are asked for)."""
    state_slot = -1
    state_slot_out = -1


class Recording:
    def __init__(self, engine, counts: Sequence[int], wants: Sequence[Sequence[int]], room: int, ring: int = 3,
                 typical_context: int = 0):
        from .. import runtime
        eng = engine                         # not kept: the engine owns its recordings
        self.counts, self.room = [int(c) for c in counts], int(room)
        n = len(self.counts)
        max_pages = [max(1, -(-room // g.page_size)) for g in eng.cache.groups]
        self.plan = eng.model.plan_step(StepShape(self.counts, None, [tuple(w) for w in wants], self.room, typical_context))
        self.layout = StepLayout(self.counts, sum(len(w) for w in wants), max_pages, eng.position_streams, self.plan.ints)
        self.total = self.layout.total
        # The host may run several steps ahead of the device: a ring of pinned buffers, each reused only
        # once the copy that read it has finished.
        self._ring = [torch.zeros(self.total, dtype=torch.int32, pin_memory=True) for _ in range(ring)]
        self._ring_events = [None] * len(self._ring)
        self._ring_at = 0
        self._dev = torch.zeros(self.total, dtype=torch.int32, device=eng.device)
        step = eng.batch_views(self._dev, self.layout, [_NoCache()] * n, [0] * n, self.room, self.plan, self.room)
        self._step = step
        self._graph = torch.cuda.CUDAGraph()
        before = runtime.launches()
        # Nothing may be freed on the device or in pinned memory while the stream is capturing, and Python's
        # collector frees what it finds whenever it runs: it does not run until the capture is over.
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self._graph):
                self.logits = eng.model.forward(step)
        finally:
            if was_enabled:
                gc.enable()
        self.graph_launches = runtime.launches() - before

    def launch(self, fill: Callable[[np.ndarray], None], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Write the step's metadata into a pinned buffer (`fill(array)`), copy it and replay the graph.
        `device_tokens` (int32 [rows] on the device): the step's token ids, laid over what the host wrote."""
        slot = self._ring_at
        self._ring_at = (slot + 1) % len(self._ring)
        if self._ring_events[slot] is not None:
            self._ring_events[slot].synchronize()
        host = self._ring[slot]
        fill(host.numpy())
        self._dev.copy_(host, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._ring_events[slot] = ev
        if device_tokens is not None:
            self._dev[:self.layout.rows].copy_(device_tokens, non_blocking=True)
        self._graph.replay()
        return self.logits

    def run(self, engine, entries, caches) -> Optional[torch.Tensor]:
        """Fill the step's metadata from the entries, copy it and replay; the logits are valid until the next run."""
        def fill(buf: np.ndarray) -> None:
            history = engine.fill_batch(buf, self.layout, entries, caches)
            self.plan.fill(history, self.layout.plan(buf))
        logits = self.launch(fill)
        engine.last_h2d_bytes = self.total * 4
        return logits
