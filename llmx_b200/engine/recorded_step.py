"""Recorded steps of any shape: prompt portions, and portions beside decoding rows.

A decode session (decode_loop.py) records the step in which every request brings one row.  The same
can be done for any pattern of row counts: the kernels a step launches, their grids and the buffers
they use depend on how many rows each request brings and on which rows' logits are wanted, not on
the requests' histories, tokens or pages, which the kernels read from the step's metadata on the
device.  A `StepRecording` holds the CUDA graph of one such pattern and the static metadata buffer
it reads; a step of the same pattern then costs one host-to-device copy and one graph launch
instead of eight kernel launches a layer from Python (about 16 us each).

The engine makes a recording of a pattern once it has seen it `EngineOptions.record_after` times
(`Engine.step(..., record=True)`): a scheduler that cuts long prompts into portions of its token
budget brings the same pattern step after step, and a benchmark that repeats a prompt length does
too.  Making a recording costs about as much as ten to twenty plain steps save, hence the wait.
"""
from __future__ import annotations

import gc
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .engine import Engine, StepEntry, StepLayout

MAX_STEP_RECORDINGS = 16   # recordings an engine keeps (least recently used goes first)
FEW_ROWS = 16              # a request with at most this many rows may run the split-KV kernel


class StepRecording:
    def __init__(self, engine: Engine, counts: Sequence[int], wants: Sequence[Sequence[int]], room: int):
        from .. import ops, ops_attn
        eng = engine                         # not kept: the engine owns its recordings
        self.counts, self.room = list(counts), room
        n = len(self.counts)
        max_pages = [max(1, -(-room // g.page_size)) for g in eng.cache.groups]
        self.layout = StepLayout(self.counts, sum(len(w) for w in wants), max_pages, extra=1)
        self._ring = [torch.zeros(self.layout.total, dtype=torch.int32, pin_memory=True) for _ in range(3)]
        self._ring_events = [None] * len(self._ring)
        self._ring_at = 0
        self._dev = torch.zeros(self.layout.total, dtype=torch.int32, device=eng.device)
        # Which requests bring few rows (split-KV kernel) and which many (prefill kernel), for every bound a
        # mixer may ask with (16 / its head ratio): constant for the pattern, so written once.
        lists = np.zeros((FEW_ROWS, n + 1), dtype=np.int32)
        split_at = []
        for m in range(1, FEW_ROWS + 1):
            few = [r for r, c in enumerate(self.counts) if c <= m]
            many = [r for r, c in enumerate(self.counts) if c > m]
            lists[m - 1, :n] = few + many
            split_at.append(len(few))
        self._lists = torch.from_numpy(lists).to(eng.device)
        # Key ranges of the split-KV kernel: the grid is fixed by the recording, the keys per range are data.
        kv_heads = max((g.spec.kv_heads for g in eng.cache.groups), default=1)
        decoding = sum(1 for c in self.counts if c <= FEW_ROWS)
        head_dim = max((g.spec.head_dim for g in eng.cache.groups), default=128)
        self.splits = ops_attn.decode_schedule(max(decoding, 1), kv_heads, room, head_dim)[0]
        step = eng._batch_views(self._dev, self.layout, [_NoCache()] * n, [0] * n, room)
        step.extras["decode_schedule"] = (self.splits, 64, self.layout.section(self._dev, len(self.layout.sizes) - 1))
        step.extras["recorded"] = True
        for m in range(1, FEW_ROWS + 1):
            k = split_at[m - 1]
            few_rows = max((c for c in self.counts if c <= m), default=0)
            many_rows = max((c for c in self.counts if c > m), default=0)
            step.extras[("attn_lists", m)] = (self._lists[m - 1, :k], k, room, few_rows, self._lists[m - 1, k:n], n - k,
                                              many_rows)
        self._step = step
        self._graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
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
        self.graph_launches = ops.launch_count() - before

    def chunk(self, context: int) -> int:
        return max(64, -(-(-(-context // 64)) // self.splits) * 64)

    def run(self, engine: Engine, entries: Sequence[StepEntry], caches) -> Optional[torch.Tensor]:
        """Fill the step's metadata, copy it and replay the graph; the logits are valid until the next run."""
        slot = self._ring_at
        self._ring_at = (slot + 1) % len(self._ring)
        if self._ring_events[slot] is not None:
            self._ring_events[slot].synchronize()
        host = self._ring[slot]
        buf = host.numpy()
        history = engine._fill_batch(buf, self.layout, entries, caches)
        few_context = max((h + c for h, c in zip(history, self.counts) if c <= FEW_ROWS), default=64)
        self.layout.section(buf, len(self.layout.sizes) - 1)[0] = self.chunk(few_context)
        self._dev.copy_(host, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._ring_events[slot] = ev
        self._graph.replay()
        from .. import ops
        ops.count_launches(self.graph_launches)
        engine.last_h2d_bytes = self.layout.total * 4
        return self.logits


class _NoCache:
    """Stands in for a request's cache while the static views are made (only the state slot is asked for)."""
    state_slot = -1
