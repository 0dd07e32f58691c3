"""Decode sessions: one token each for a set of live requests, recorded once and replayed.

This is the inner loop of generation once prompts are in the cache.  The work of such a step has
the same shape every time (same rows, same kernels, same grids), so it is recorded in a CUDA graph
(recording.py) and replayed: a step then costs one host-to-device copy of the step's metadata and one graph
launch instead of several hundred kernel launches.

A recording depends on two numbers only: how many requests decode, and how many tokens of context
its block tables have room for (in steps of 2,048 tokens).  The engine keeps the recordings it has
made, so a session over other requests -- one has finished, another has joined -- finds its
recording ready; a session only keeps the host's copy of its requests' metadata.  The first
decode step at a new batch size runs through `Engine.step`, which also loads and warms the
kernels that the recording will hold.
"""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from . import batch as B
from .engine import Engine, StepEntry, StepError, room_for
from .recording import Recording

MAX_RECORDINGS = 32        # decode recordings an engine keeps (least recently used goes first)


def recording_of(engine: Engine, b: int, room: int, make: bool = True) -> Optional[Recording]:
    """The engine's recording for (`b`, `room`), made now if there is none (unless `make` is false)."""
    kept = engine.decode_recordings
    rec = kept.get((b, room))
    if rec is not None:
        kept.move_to_end((b, room))
        return rec
    if not make:
        return None
    rec = Recording(engine, [1] * b, [(0,)] * b, room, ring=4)
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
        self._rec: Optional[Recording] = None
        for rid in self.request_ids:
            if rid not in engine.cache.live:
                raise StepError(f"request {rid!r} is not live; a decode session continues requests that are")

    def _fill(self, host: np.ndarray, tokens: Sequence[int], caches) -> None:
        """Write the step's metadata into `host`.  The master copy is kept between steps and only what a step
        changes is touched: tokens, positions, slots, and a block-table row when a request's pages have changed."""
        b = len(caches)
        rec = self._rec
        lay = rec.layout
        m = self._master
        hist = [rc.length for rc in caches]
        if not self._master_ready:
            lay.section(m, B.ROW_REQUEST)[:] = np.arange(b)
            lay.section(m, B.ROW_START)[:] = np.arange(b)
            lay.section(m, B.ROW_COUNT)[:] = 1
            lay.section(m, B.LOGIT_ROWS)[:] = np.arange(b)
            self._pages_seen = [[(0, -2)] * b for _ in self.engine.cache.groups]
            self._master_ready = True
        lay.section(m, B.TOKENS)[:] = tokens
        lay.section(m, B.POSITIONS).reshape(lay.streams, b)[:] = hist
        lay.section(m, B.HISTORY)[:] = hist
        lay.section(m, B.STATE_SLOTS)[:] = [rc.state_slot for rc in caches]
        lay.section(m, B.STATE_SLOTS_OUT)[:] = [rc.state_slot_out for rc in caches]
        for g, grp in enumerate(self.engine.cache.groups):
            ps = grp.page_size
            bt, sl = lay.tables(m, g), lay.slots(m, g)
            seen = self._pages_seen[g]
            for r, rc in enumerate(caches):
                pages = rc.tables[g].pages
                mark = (len(pages), pages[-1])
                if seen[r] != mark:          # a new page, or (after a step that failed) another page at the same length
                    bt[r, :len(pages)] = pages          # released pages (-1) are never addressed
                    seen[r] = mark
                sl[r] = pages[hist[r] // ps] * ps + hist[r] % ps
        rec.plan.fill(hist, lay.plan(m))
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
                logits = rec.launch(lambda host: self._fill(host, host_tokens, caches), device_tokens)
        except BaseException:
            for rc in prepared:
                rc.abort()
            raise
        for rc in caches:
            rc.commit()
        eng.steps_run += 1
        from .. import runtime
        self.graph_launches = rec.graph_launches
        runtime.count_launches(rec.graph_launches)
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
