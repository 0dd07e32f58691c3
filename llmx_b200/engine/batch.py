"""A step's metadata: one int32 buffer, filled on the host, copied once, viewed by the kernels.

`StepLayout` says where each section lies; `fill` writes a buffer for given requests; `views` makes the
`StepBatch` (torch views for parts written in Python, an `llmx_step` for the native runtime) over a device copy.
The reference builds the same lists per pass (src/model/passes.hpp:334-393; the device backends flatten block
tables and row ranges into one uploaded array, src/backends/gpu/backend_core.hpp:1841-1881).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import runtime
from ..parts.base import GroupView, StepBatch

TOKENS, POSITIONS, ROW_REQUEST, ROW_START, ROW_COUNT, HISTORY, STATE_SLOTS, LOGIT_ROWS, STATE_SLOTS_OUT, FIRST_GROUP = range(10)


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class StepLayout:
    """Where a step's metadata lies in its one int32 buffer (sections padded to 16 bytes):
    0 token ids [rows], 1 positions [streams, rows], 2 request of each row [rows], 3 first row [requests],
    4 row count [requests], 5 history [requests], 6 state slots read [requests], 7 rows whose logits are wanted,
    8 state slots written [requests], then for every cache group its block tables [requests, max_pages] and the rows' cache slots [rows],
    then the ints of the parts' launch plans."""

    def __init__(self, counts: Sequence[int], wanted: int, max_pages: Sequence[int], streams: int = 1, plan_ints: int = 0):
        self.counts = [int(c) for c in counts]
        self.requests, self.rows, self.wanted = len(self.counts), sum(self.counts), int(wanted)
        self.max_pages = [int(m) for m in max_pages]
        self.streams = max(int(streams), 1)
        self.plan_ints = int(plan_ints)
        self.starts = [0] * self.requests
        for r in range(1, self.requests):
            self.starts[r] = self.starts[r - 1] + self.counts[r - 1]
        self.sizes = [self.rows, self.streams * self.rows, self.rows, self.requests, self.requests, self.requests,
                      self.requests, self.wanted, self.requests]
        for mp in self.max_pages:
            self.sizes += [self.requests * mp, self.rows]
        self.plan_section = len(self.sizes)
        self.sizes.append(self.plan_ints)
        self.offsets, at = [], 0
        for size in self.sizes:
            self.offsets.append(at)
            at += _pad4(max(size, 1))
        self.total = at

    def section(self, buf, i: int):
        return buf[self.offsets[i]:self.offsets[i] + self.sizes[i]]

    def tables(self, buf, g: int):
        return self.section(buf, FIRST_GROUP + 2 * g).reshape(self.requests, self.max_pages[g])

    def slots(self, buf, g: int):
        return self.section(buf, FIRST_GROUP + 2 * g + 1)

    def plan(self, buf):
        return self.section(buf, self.plan_section)


def fill(buf: np.ndarray, layout: StepLayout, tokens: Sequence[Sequence[int]], histories: Sequence[int],
         state_slots: Sequence[int], wants: Sequence[Sequence[int]], pages: Sequence[Sequence[Sequence[int]]],
         page_sizes: Sequence[int], more_positions: Optional[Sequence[Optional[Sequence[Sequence[int]]]]] = None,
         state_slots_out: Optional[Sequence[int]] = None) -> None:
    """Write the metadata of a step into `buf` (int32, `layout.total` values).  `pages[g][r]`: request r's page ids
    in cache group g; `more_positions[r]` (optional): the request's rows' positions in streams 1.. (stream 0 is the
    position in the request; absent streams repeat it)."""
    buf[:] = 0
    tok, rreq = layout.section(buf, TOKENS), layout.section(buf, ROW_REQUEST)
    pos = layout.section(buf, POSITIONS).reshape(layout.streams, layout.rows)
    for r in range(layout.requests):
        a, n = layout.starts[r], layout.counts[r]
        tok[a:a + n] = np.asarray(tokens[r], dtype=np.int64)
        own = np.arange(histories[r], histories[r] + n)
        pos[:, a:a + n] = own
        extra = more_positions[r] if more_positions is not None else None
        if extra is not None:
            for k, stream in enumerate(extra):
                pos[1 + k, a:a + n] = np.asarray(stream, dtype=np.int64)
        rreq[a:a + n] = r
    layout.section(buf, ROW_START)[:] = layout.starts
    layout.section(buf, ROW_COUNT)[:] = layout.counts
    layout.section(buf, HISTORY)[:] = histories
    layout.section(buf, STATE_SLOTS)[:] = state_slots
    layout.section(buf, STATE_SLOTS_OUT)[:] = state_slots if state_slots_out is None else state_slots_out
    lr, k = layout.section(buf, LOGIT_ROWS), 0
    for r, want in enumerate(wants):
        for w in want:
            lr[k] = layout.starts[r] + int(w)
            k += 1
    for g, ps in enumerate(page_sizes):
        bt, sl = layout.tables(buf, g), layout.slots(buf, g)
        for r in range(layout.requests):
            pg = pages[g][r]
            bt[r, :len(pg)] = pg
            parr = np.asarray(pg, dtype=np.int64)
            p = np.arange(histories[r], histories[r] + layout.counts[r])
            a = layout.starts[r]
            # A released page (-1) is never addressed: the window keeps queries above it.
            sl[a:a + layout.counts[r]] = parr[p // ps] * ps + p % ps


def views(dev: torch.Tensor, layout: StepLayout, caches, page_sizes: Sequence[int], histories: Sequence[int],
          state_slots: Sequence[int], max_context: int, plan=None, room: int = 0,
          state_slots_out: Optional[Sequence[int]] = None) -> StepBatch:
    """The StepBatch whose device tensors are the sections of `dev` (the device copy of a filled buffer)."""
    n_req = layout.requests
    groups = [GroupView(layout.tables(dev, g), layout.slots(dev, g), ps) for g, ps in enumerate(page_sizes)]
    streams = layout.section(dev, POSITIONS).view(layout.streams, layout.rows)
    s = runtime.StepStruct()
    s.rows, s.requests, s.wanted, s.groups = layout.rows, n_req, layout.wanted, len(groups)
    s.position_streams, s.room = layout.streams, int(room)
    s.meta = dev.data_ptr()
    o = layout.offsets
    (s.token_ids, s.positions, s.row_request, s.row_start, s.row_count, s.history, s.state_slots, s.logit_rows,
     s.state_slots_out) = o[:9]
    if len(groups) > runtime.MAX_GROUPS:
        raise runtime.KernelError(f"a model may have {runtime.MAX_GROUPS} cache groups at most")
    for g, ps in enumerate(page_sizes):
        s.block_tables[g], s.table_stride[g] = o[FIRST_GROUP + 2 * g], layout.max_pages[g]
        s.slots[g], s.page_size[g] = o[FIRST_GROUP + 2 * g + 1], ps
    s.plan_offset = o[layout.plan_section]
    s.caches = caches.views.handle if caches is not None and getattr(caches, "views", None) is not None else None
    s.error_word = runtime.error_word(dev.device).data_ptr()
    s.counters = runtime.counters(dev.device).data_ptr()
    s.stream = runtime.current_stream()
    if plan is not None:
        plan.base = o[layout.plan_section]
        plan.device = layout.plan(dev)
    return StepBatch(rows=layout.rows, requests=n_req, token_ids=layout.section(dev, TOKENS), positions=streams[0],
                     row_request=layout.section(dev, ROW_REQUEST), row_start=layout.section(dev, ROW_START),
                     row_count=layout.section(dev, ROW_COUNT), history=layout.section(dev, HISTORY),
                     state_slots=layout.section(dev, STATE_SLOTS), logit_rows=layout.section(dev, LOGIT_ROWS),
                     groups=groups, caches=caches, host_row_start=list(layout.starts), host_row_count=list(layout.counts),
                     host_history=list(histories), host_state_slots=list(state_slots),
                     state_slots_out=layout.section(dev, STATE_SLOTS_OUT),
                     host_state_slots_out=list(state_slots if state_slots_out is None else state_slots_out),
                     max_row_count=max(layout.counts),
                     max_context=max_context, position_streams=streams, struct=s, plan=plan, room=int(room))


def single_group_step(device, layout_rows: Sequence[tuple], tables: np.ndarray, page_size: int, caches=None,
                      plan_parts: Sequence[int] = (), wants: Sequence[Sequence[int]] = ()) -> StepBatch:
    """A step over one cache group from (history, rows) pairs and ready block tables [requests, max_pages]:
    what the kernel tests hand the attention kernels.  `plan_parts`: native part handles to plan for."""
    from ..parts.attention import NativePlan
    from ..parts.base import StepShape
    from ..models.model import ModelPlan
    counts = [n for _, n in layout_rows]
    histories = [h for h, _ in layout_rows]
    plan = None
    if plan_parts:
        native = NativePlan(None, list(plan_parts), StepShape(counts, histories))
        plan = ModelPlan(native if native.ints else None, [])
    layout = StepLayout(counts, sum(len(w) for w in wants), [tables.shape[1]], 1, plan.ints if plan else 0)
    host = torch.zeros(layout.total, dtype=torch.int32)
    buf = host.numpy()
    pages = [[list(tables[r]) for r in range(len(counts))]]
    fill(buf, layout, [[0] * n for n in counts], histories, [-1] * len(counts), wants or [()] * len(counts), pages, [page_size])
    if plan is not None:
        plan.fill(histories, layout.plan(buf))
    dev = host.to(device)
    return views(dev, layout, caches, [page_size], histories, [-1] * len(counts),
                 max(h + n for h, n in layout_rows), plan)


def step_from_requests(manager, request_caches, counts: Sequence[int], device, parts: Sequence = (),
                       wants: Optional[Sequence[Sequence[int]]] = None, tokens: Optional[Sequence[Sequence[int]]] = None,
                       streams: int = 1) -> StepBatch:
    """A step for live requests of a cache manager (each prepared for `counts[r]` more tokens), planned for the given
    parts: what `Engine.step` builds, for callers that run single parts."""
    from ..models.model import ModelPlan
    from ..parts.attention import NativePlan
    from ..parts.base import StepShape
    histories = [rc.length for rc in request_caches]
    wants = wants if wants is not None else [()] * len(counts)
    shape = StepShape(list(counts), histories, wants)
    handles = [p.native for p in parts if getattr(p, "native_planned", False)]
    native = NativePlan(None, handles, shape) if handles else None
    python = [(p, pl) for p in parts if not getattr(p, "native_planned", False) for pl in [p.plan_step(shape)] if pl is not None and pl.ints]
    plan = ModelPlan(native if native is not None and native.ints else None, python)
    n_groups = len(manager.groups)
    max_pages = [max(1, max(len(rc.tables[g].pages) for rc in request_caches)) for g in range(n_groups)]
    layout = StepLayout(counts, sum(len(w) for w in wants), max_pages, streams, plan.ints)
    host = torch.zeros(layout.total, dtype=torch.int32)
    buf = host.numpy()
    pages = [[rc.tables[g].pages for rc in request_caches] for g in range(n_groups)]
    page_sizes = [g.page_size for g in manager.groups]
    fill(buf, layout, tokens if tokens is not None else [[0] * n for n in counts], histories,
         [rc.state_slot for rc in request_caches], wants, pages, page_sizes, None, [rc.state_slot_out for rc in request_caches])
    plan.fill(histories, layout.plan(buf))
    dev = host.to(device)
    return views(dev, layout, manager, page_sizes, histories, [rc.state_slot for rc in request_caches],
                 max(h + n for h, n in zip(histories, counts)), plan, 0, [rc.state_slot_out for rc in request_caches])
