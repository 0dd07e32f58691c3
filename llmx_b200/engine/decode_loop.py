"""A decode session: a fixed set of live requests, one token each per step, recorded once and replayed.

This is the inner loop of generation once prompts are in the cache.  The work of such a step has
the same shape every time (same rows, same kernels, same grids), so the session records it in a
CUDA graph and replays it: a step then costs one host-to-device copy of the step's metadata and
one graph launch instead of several hundred kernel launches.  What the session runs is the
model's own forward pass over the engine's own cache; what changes from step to step (token ids,
positions, cache slots, block tables, the keys per range of the split-KV kernel) lives in one
device buffer the kernels read.

The graph is recorded again when a request outgrows the block-table width or the key ranges it
was recorded for.  The first step of a session always runs through `Engine.step` (it also warms
the kernels up).
"""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import GroupView, StepBatch
from .engine import Engine, StepEntry, StepError, _pad4


class DecodeSession:
    GROWTH = 2048          # tokens of room a recording leaves before it must be made again

    def __init__(self, engine: Engine, request_ids: Sequence[Hashable], use_graph: bool = True):
        self.engine = engine
        self.request_ids = list(request_ids)
        self.use_graph = use_graph and engine.model.recordable
        self.h2d_bytes_per_step = 0
        self.graph_launches = 0          # kernels one replay launches
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._steps = 0
        for rid in self.request_ids:
            if rid not in engine.cache.live:
                raise StepError(f"request {rid!r} is not live; a decode session continues requests that are")

    # -- layout of the static metadata buffer -----------------------------------------------
    def _layout(self, max_pages: List[int]):
        b = len(self.request_ids)
        sizes = [b, b, b, b, b, b, b, b, b + 1, 1]    # tokens, positions, row_request, row_start, row_count, history,
        #                                               state slots, logit rows, request list, keys per range
        for mp in max_pages:
            sizes += [b * mp, b]
        offsets, at = [], 0
        for s in sizes:
            offsets.append(at)
            at += _pad4(s)
        return sizes, offsets, at

    def _fill(self, host: np.ndarray, tokens: Sequence[int], caches, chunk: int) -> None:
        """Write the step's metadata into `host`.  The master copy is kept between steps and only what a step
        changes is touched: tokens, positions, slots, and a block-table entry when a request enters a new page."""
        b = len(caches)
        sizes, offsets = self._sizes, self._offsets
        m = self._master

        def sec(i):
            return m[offsets[i]:offsets[i] + sizes[i]]
        hist = [rc.length for rc in caches]
        if not self._master_ready:
            sec(2)[:] = np.arange(b)
            sec(3)[:] = np.arange(b)
            sec(4)[:] = 1
            sec(6)[:] = [rc.state_slot for rc in caches]
            sec(7)[:] = np.arange(b)
            sec(8)[:b] = np.arange(b)
            self._pages_seen = [[0] * b for _ in self.engine.cache.groups]
            self._master_ready = True
        sec(0)[:] = tokens
        sec(1)[:] = hist
        sec(5)[:] = hist
        sec(9)[0] = chunk
        for g, grp in enumerate(self.engine.cache.groups):
            ps = grp.page_size
            mp = self._max_pages[g]
            bt = sec(10 + 2 * g).reshape(b, mp)
            sl = sec(11 + 2 * g)
            seen = self._pages_seen[g]
            for r, rc in enumerate(caches):
                pages = rc.tables[g].pages
                if seen[r] != len(pages):
                    bt[r, :len(pages)] = pages          # released pages (-1) are never addressed
                    seen[r] = len(pages)
                sl[r] = pages[hist[r] // ps] * ps + hist[r] % ps
        host[:] = m

    def _record(self, caches) -> None:
        from .. import ops, ops_attn
        eng = self.engine
        b = len(caches)
        ctx_now = max(rc.length + rc.pending for rc in caches)
        room = min(ctx_now + self.GROWTH, eng.max_positions)
        self._max_pages = [max(1, -(-room // g.page_size)) for g in eng.cache.groups]
        self._sizes, self._offsets, total = self._layout(self._max_pages)
        # The host may run several steps ahead of the device: a ring of pinned buffers, each reused only
        # once the copy that read it has finished.
        self._ring = [torch.zeros(total, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._ring_events = [None] * len(self._ring)
        self._ring_at = 0
        self._dev = torch.zeros(total, dtype=torch.int32, device=eng.device)
        self._master = np.zeros(total, dtype=np.int32)
        self._master_ready = False
        self._room = room
        # Key ranges of the split-KV kernel: the grid is fixed by the recording, the keys per range are data.
        kv_heads = max((g.spec.kv_heads for g in eng.cache.groups), default=1)
        self._splits, _ = ops_attn.decode_schedule(b, kv_heads, room)

        def dsec(i):
            return self._dev[self._offsets[i]:self._offsets[i] + self._sizes[i]]
        groups = [GroupView(dsec(10 + 2 * g).view(b, self._max_pages[g]), dsec(11 + 2 * g), grp.page_size)
                  for g, grp in enumerate(eng.cache.groups)]
        step = StepBatch(rows=b, requests=b, token_ids=dsec(0), positions=dsec(1), row_request=dsec(2),
                         row_start=dsec(3), row_count=dsec(4), history=dsec(5), state_slots=dsec(6),
                         logit_rows=dsec(7), groups=groups, caches=eng.cache, host_row_start=list(range(b)),
                         host_row_count=[1] * b, host_history=[0] * b, max_row_count=1, max_context=room)
        chunk_dev = dsec(9)
        step.extras["decode_schedule"] = (self._splits, 64, chunk_dev)
        step.extras["recorded"] = True
        for ratio_rows in range(1, 17):       # every mixer's list of "requests with few rows" is all of them
            step.extras[("attn_lists", ratio_rows)] = (dsec(8)[:b], b, room, 1, dsec(8)[b:b], 0, 0)
        self._step = step
        self._graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(self._graph):
            self._logits = eng.model.forward(step)
        self.graph_launches = ops.launch_count() - before

    def _chunk(self, ctx: int) -> int:
        return max(64, -(-(-(-ctx // 64)) // self._splits) * 64)

    def step(self, tokens: Sequence[int]) -> torch.Tensor:
        """Feed one token per request (in the session's order); float32 logits [requests, vocab] on the
        device, valid until the next step."""
        eng = self.engine
        if len(tokens) != len(self.request_ids):
            raise StepError("a decode step needs one token for every request of the session")
        self._steps += 1
        if not self.use_graph or self._steps == 1:
            logits = eng.step([StepEntry(rid, [int(t)], [0]) for rid, t in zip(self.request_ids, tokens)])
            self.h2d_bytes_per_step = eng.last_h2d_bytes
            return logits
        caches = [eng.cache.live[rid] for rid in self.request_ids]
        for t, rc in zip(tokens, caches):
            if not 0 <= int(t) < eng.model.vocab_size:
                raise StepError(f"token id {t} is outside the vocabulary of {eng.model.vocab_size}")
            if rc.length + 1 > eng.max_positions:
                raise StepError(f"request {rc.request_id!r}: context length of {eng.max_positions} exceeded")
        prepared = []
        try:
            for rc in caches:
                rc.prepare(1)
                prepared.append(rc)
            ctx = max(rc.length + 1 for rc in caches)
            with torch.cuda.device(eng.device):
                if self._graph is None or ctx > self._room:
                    self._record(caches)
                slot = self._ring_at
                self._ring_at = (slot + 1) % len(self._ring)
                if self._ring_events[slot] is not None:
                    self._ring_events[slot].synchronize()
                host = self._ring[slot]
                self._fill(host.numpy(), [int(t) for t in tokens], caches, self._chunk(ctx))
                self._dev.copy_(host, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                self._ring_events[slot] = ev
                self._graph.replay()
        except BaseException:
            for rc in prepared:
                rc.abort()
            raise
        for rc in caches:
            rc.commit()
        eng.steps_run += 1
        from .. import ops
        ops.count_launches(self.graph_launches)
        self.h2d_bytes_per_step = self._dev.numel() * 4
        return self._logits

    def close(self) -> None:
        self._graph = None
        self._logits = None
        self._step = None
