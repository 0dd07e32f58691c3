"""Decode sessions and recordings: one token each for a set of live requests, recorded once and replayed.

This is the inner loop of generation once prompts are in the cache.  The work of such a step has
the same shape every time (same rows, same kernels, same grids), so it is recorded in a CUDA graph
and replayed: a step then costs one host-to-device copy of the step's metadata and one graph
launch instead of several hundred kernel launches.  What is recorded is the model's own forward
pass over the engine's own cache; what changes from step to step (token ids, positions, cache
slots, block tables, the keys per range of the split-KV kernel) lives in one device buffer the
kernels read.

A recording depends on two numbers only: how many requests decode, and how many tokens of context
its block tables have room for (in steps of 2,048 tokens).  The engine keeps the recordings it has
made, so a session over other requests -- one has finished, another has joined -- finds its
recording ready; a session only keeps the host's copy of its requests' metadata.  The first
decode step at a new batch size runs through `Engine.step`, which also loads and warms the
kernels that the recording will hold.
"""
from __future__ import annotations

import gc
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import GroupView, StepBatch
from .engine import Engine, StepEntry, StepError, _pad4, room_for

MAX_RECORDINGS = 32        # recordings an engine keeps (least recently used goes first)


class DecodeRecording:
    """The graph of one decode step for `b` requests with room for `room` tokens of context each, and the
    buffers it reads its metadata from."""

    def __init__(self, engine: Engine, b: int, room: int):
        from .. import ops, ops_attn
        eng = engine                     # not kept: the engine owns its recordings, not the other way round
        self.b, self.room = b, room
        self.max_pages = [max(1, -(-room // g.page_size)) for g in eng.cache.groups]
        self.sizes, self.offsets, self.total = self._layout(b, self.max_pages)
        # The host may run several steps ahead of the device: a ring of pinned buffers, each reused only
        # once the copy that read it has finished.
        self._ring = [torch.zeros(self.total, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._ring_events = [None] * len(self._ring)
        self._ring_at = 0
        self._dev = torch.zeros(self.total, dtype=torch.int32, device=eng.device)
        # Key ranges of the split-KV kernel: the grid is fixed by the recording, the keys per range are data.
        kv_heads = max((g.spec.kv_heads for g in eng.cache.groups), default=1)
        head_dim = max((g.spec.head_dim for g in eng.cache.groups), default=128)
        self.splits, _ = ops_attn.decode_schedule(b, kv_heads, room, head_dim)

        def dsec(i):
            return self._dev[self.offsets[i]:self.offsets[i] + self.sizes[i]]
        groups = [GroupView(dsec(10 + 2 * g).view(b, self.max_pages[g]), dsec(11 + 2 * g), grp.page_size)
                  for g, grp in enumerate(eng.cache.groups)]
        step = StepBatch(rows=b, requests=b, token_ids=dsec(0), positions=dsec(1), row_request=dsec(2),
                         row_start=dsec(3), row_count=dsec(4), history=dsec(5), state_slots=dsec(6),
                         logit_rows=dsec(7), groups=groups, caches=eng.cache, host_row_start=list(range(b)),
                         host_row_count=[1] * b, host_history=[0] * b, max_row_count=1, max_context=room)
        step.extras["decode_schedule"] = (self.splits, 64, dsec(9))
        step.extras["recorded"] = True
        for ratio_rows in range(1, 17):       # every mixer's list of "requests with few rows" is all of them
            step.extras[("attn_lists", ratio_rows)] = (dsec(8)[:b], b, room, 1, dsec(8)[b:b], 0, 0)
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

    @staticmethod
    def _layout(b: int, max_pages: List[int]):
        sizes = [b, b, b, b, b, b, b, b, b + 1, 1]    # tokens, positions, row_request, row_start, row_count, history,
        #                                               state slots, logit rows, request list, keys per range
        for mp in max_pages:
            sizes += [b * mp, b]
        offsets, at = [], 0
        for s in sizes:
            offsets.append(at)
            at += _pad4(s)
        return sizes, offsets, at

    def chunk(self, ctx: int) -> int:
        return max(64, -(-(-(-ctx // 64)) // self.splits) * 64)

    def launch(self, fill, device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Copy the step's metadata (written into a pinned buffer by `fill(array)`) and replay the graph.
        `device_tokens` (int32 [b] on the device): the step's token ids, laid over what the host wrote."""
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
            self._dev[:self.b].copy_(device_tokens, non_blocking=True)
        self._graph.replay()
        return self.logits


def recording_of(engine: Engine, b: int, room: int, make: bool = True) -> Optional[DecodeRecording]:
    """The engine's recording for (`b`, `room`), made now if there is none (unless `make` is false)."""
    kept = engine.decode_recordings
    rec = kept.get((b, room))
    if rec is not None:
        kept.move_to_end((b, room))
        return rec
    if not make:
        return None
    rec = DecodeRecording(engine, b, room)
    kept[(b, room)] = rec
    while len(kept) > MAX_RECORDINGS:
        kept.popitem(last=False)
    return rec


class DecodeSession:
    def __init__(self, engine: Engine, request_ids: Sequence[Hashable], use_graph: bool = True,
                 plain_steps: int = 1):
        """`plain_steps`: how many steps a session runs through `Engine.step` before it has a missing
        recording made (at least the one that warms a new batch size up).  Making a recording costs about
        as much as ten to twenty plain steps, so a caller whose sessions may be short asks for a few."""
        self.engine = engine
        self.plain_steps = max(1, int(plain_steps))
        self._plain_run = 0
        self.request_ids = list(request_ids)
        self.use_graph = use_graph and engine.model.recordable
        self.h2d_bytes_per_step = 0
        self.graph_launches = 0          # kernels one replay launches
        self._rec: Optional[DecodeRecording] = None
        for rid in self.request_ids:
            if rid not in engine.cache.live:
                raise StepError(f"request {rid!r} is not live; a decode session continues requests that are")

    def _fill(self, host: np.ndarray, tokens: Sequence[int], caches, chunk: int) -> None:
        """Write the step's metadata into `host`.  The master copy is kept between steps and only what a step
        changes is touched: tokens, positions, slots, and a block-table entry when a request enters a new page."""
        b = len(caches)
        rec = self._rec
        sizes, offsets = rec.sizes, rec.offsets
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
            mp = rec.max_pages[g]
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

    def step(self, tokens) -> torch.Tensor:
        """Feed one token per request (in the session's order); float32 logits [requests, vocab] on the
        device, valid until the next step.  `tokens`: a sequence of ids, or an int32 tensor on the device
        (what the sampler drew for the step before: the host then need not have seen the ids yet)."""
        eng = self.engine
        b = len(self.request_ids)
        if len(tokens) != b:
            raise StepError("a decode step needs one token for every request of the session")
        device_tokens = tokens if isinstance(tokens, torch.Tensor) else None
        caches = [eng.cache.live[rid] for rid in self.request_ids]
        ctx = max(rc.length + 1 for rc in caches)
        room = room_for(ctx, eng.max_positions)
        warmed = eng.decode_warmed
        have = recording_of(eng, b, room, make=False) is not None
        if not self.use_graph or (not have and (b not in warmed or self._plain_run < self.plain_steps)):
            if device_tokens is not None:
                tokens = device_tokens.cpu().tolist()          # a plain step builds its batch on the host
            logits = eng.step([StepEntry(rid, [int(t)], [0]) for rid, t in zip(self.request_ids, tokens)])
            warmed.add(b)
            self._plain_run += 1
            self.h2d_bytes_per_step = eng.last_h2d_bytes
            return logits
        host_tokens = [0] * b if device_tokens is not None else [int(t) for t in tokens]
        for t, rc in zip(host_tokens, caches):
            if not 0 <= t < eng.model.vocab_size:
                raise StepError(f"token id {t} is outside the vocabulary of {eng.model.vocab_size}")
            if rc.length + 1 > eng.max_positions:
                raise StepError(f"request {rc.request_id!r}: context length of {eng.max_positions} exceeded")
        prepared = []
        try:
            for rc in caches:
                rc.prepare(1)
                prepared.append(rc)
            with torch.cuda.device(eng.device):
                rec = recording_of(eng, b, room)
                if rec is not self._rec:
                    self._rec = rec
                    self._master = np.zeros(rec.total, dtype=np.int32)
                    self._master_ready = False
                logits = rec.launch(lambda host: self._fill(host, host_tokens, caches, rec.chunk(ctx)), device_tokens)
        except BaseException:
            for rc in prepared:
                rc.abort()
            raise
        for rc in caches:
            rc.commit()
        eng.steps_run += 1
        from .. import ops
        self.graph_launches = rec.graph_launches
        ops.count_launches(rec.graph_launches)
        self.h2d_bytes_per_step = rec.total * 4
        return logits

    def replays(self) -> bool:
        """Whether the next step replays a recording (and so can take its tokens from the device)."""
        if not self.use_graph:
            return False
        eng = self.engine
        ctx = max(eng.cache.live[rid].length + 1 for rid in self.request_ids)
        return recording_of(eng, len(self.request_ids), room_for(ctx, eng.max_positions), make=False) is not None

    def close(self) -> None:
        """The session is over.  Its recording stays with the engine for the next session of its size."""
        self._rec = None
