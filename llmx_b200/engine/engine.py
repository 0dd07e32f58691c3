"""The engine: a loaded model, its cache, and the one step function.

`Engine.step(entries)` is everything between a batch of (request, its next
tokens) and the logits at the wanted places.  A batch may mix portions of
prompts with single decoded tokens, cut anywhere; the step runs only the tokens
it is given, from the cache earlier steps left, as one batch.  It is the
counterpart of the reference's `Model::forward` (src/model/passes.hpp:13-25,
batch layout :271-413) and keeps its transaction rule: pages are prepared
before the step, committed after it, and a step that fails leaves every request
where it was (src/model/passes.hpp:1124-1134).

Generation (`llmx_b200.engine.generate`), the scheduler, the command line and
`bin/trace_run` all drive this same function.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from collections import OrderedDict
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import CacheExhausted, RELEASED
from ..parts.base import GroupView, Precision, StepBatch
from ..registry import architecture_of, config_from_dir
from ..weights.safetensors import TensorDirectory


class StepError(ValueError):
    """A batch the step refuses before any work."""


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places whose logits are wanted."""
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"
    kv_tokens: int = 8192            # tokens the cache pool is made for
    page_size: int = 16
    max_requests: int = 64           # live requests (state slots; block-table rows)
    device: str = "cuda:0"
    record_after: int = 16           # plain steps of one shape before `step(..., record=True)` records it: making
    #                                  a recording costs about as much as ten to twenty plain steps save
    yarn: Optional[float] = None     # the rope scaled by YaRN at this factor, whatever the files say (--yarn)
    yarn_original_ctx: Optional[int] = None   # the trained length `yarn` scales from (default: the files')


def _scaled(config, options: "EngineOptions"):
    """The configuration with the rope scaling the options force on it, if any."""
    if options.yarn is None:
        if options.yarn_original_ctx is not None:
            raise StepError("yarn_original_ctx is the length `yarn` scales from; give `yarn`")
        return config
    if not hasattr(config, "with_yarn"):
        raise StepError(f"{type(config).__name__} has no rope that YaRN could scale")
    return config.with_yarn(options.yarn, options.yarn_original_ctx)


def _pad4(n: int) -> int:
    return (n + 3) & ~3


ROOM_STEP = 2048           # a recording's room for context is a multiple of this


def room_for(context: int, max_positions: int) -> int:
    """Tokens of context a recorded step at `context` tokens has room for: at least one `ROOM_STEP`
    ahead, so that recordings change rarely."""
    return min((context // ROOM_STEP + 2) * ROOM_STEP, max(max_positions, 1))


class StepLayout:
    """Where a step's metadata lies in its one int32 buffer (sections padded to 16 bytes):
    0 token ids [rows], 1 positions [rows], 2 request of each row [rows], 3 first row [requests],
    4 row count [requests], 5 history [requests], 6 state slots [requests], 7 rows whose logits are wanted,
    then for every cache group its block tables [requests, max_pages] and the rows' cache slots [rows],
    then `extra` ints (a recorded step keeps the keys per range of the split-KV kernel there)."""

    def __init__(self, counts: Sequence[int], wanted: int, max_pages: Sequence[int], extra: int = 0):
        self.counts = [int(c) for c in counts]
        self.requests, self.rows, self.wanted = len(self.counts), sum(self.counts), wanted
        self.max_pages = list(max_pages)
        self.starts = [0] * self.requests
        for r in range(1, self.requests):
            self.starts[r] = self.starts[r - 1] + self.counts[r - 1]
        self.sizes = [self.rows, self.rows, self.rows, self.requests, self.requests, self.requests, self.requests, wanted]
        for mp in self.max_pages:
            self.sizes += [self.requests * mp, self.rows]
        if extra:
            self.sizes.append(extra)
        self.offsets, at = [], 0
        for size in self.sizes:
            self.offsets.append(at)
            at += _pad4(max(size, 1))
        self.total = at

    def section(self, buf, i: int):
        return buf[self.offsets[i]:self.offsets[i] + self.sizes[i]]


class Engine:
    def __init__(self, model, options: EngineOptions):
        """`model` must be loaded (`Model.load`) on `options.device` in `options.dtype`."""
        if not torch.cuda.is_available():
            raise RuntimeError("llmx_b200 runs on a CUDA device; none is available (there is no CPU path)")
        self.model = model
        self.options = options
        self.device = torch.device(options.device)
        self.precision = Precision.of(options.dtype)
        if model.precision is None or model.precision.act is not self.precision.act:
            raise ValueError("the model was not loaded in the engine's dtype")
        self.max_positions = model.max_positions
        self.cache = CacheManager(model.cache_entry_specs(), options.page_size, options.kv_tokens,
                                  options.max_requests, kv_dtype=self.precision.act, device=self.device)
        model.prepare(min(self.max_positions, max(options.kv_tokens, 1)), self.device)
        self.steps_run = 0
        # Recorded decode steps by (requests, room for context), least recently used first, and the batch
        # sizes whose kernels a plain step has already run (see decode_loop.py).
        self.decode_recordings = OrderedDict()
        self.decode_warmed = set()
        # Recorded steps of other shapes by (rows per request, wanted places, room), and how often a shape
        # that has no recording yet has come (see recorded_step.py).
        self.step_recordings = OrderedDict()
        self._shapes_seen: Dict[tuple, int] = {}
        self.last_h2d_bytes = 0

    # -- construction ------------------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir: str, options: Optional[EngineOptions] = None) -> "Engine":
        """Load a folder with config.json and safetensors; the model class is chosen by config.json."""
        options = options or EngineOptions()
        entry, config = config_from_dir(model_dir)
        config = _scaled(config, options)
        model = entry.build(config)
        source = TensorDirectory(model_dir)
        with torch.cuda.device(torch.device(options.device)):
            model.load(source, torch.device(options.device), Precision.of(options.dtype), where=model_dir)
        source.close()
        return cls(model, options)

    @classmethod
    def from_config(cls, config, seed: int, options: Optional[EngineOptions] = None) -> "Engine":
        """A model of `config` with random weights made on the device (no files)."""
        from ..weights.random_init import RandomSource
        options = options or EngineOptions()
        config = _scaled(config, options)
        entry = architecture_of(config.to_dict())
        model = entry.build(config)
        src = RandomSource(model.tensor_specs(), seed, dtype=torch.bfloat16, device=options.device, skip_optional=True)
        model.load(src, torch.device(options.device), Precision.of(options.dtype), where="random weights")
        return cls(model, options)

    # -- requests ------------------------------------------------------------------
    def length(self, request_id: Hashable) -> int:
        rc = self.cache.live.get(request_id)
        return rc.length if rc else 0

    def end(self, request_id: Hashable) -> None:
        """The request is finished: what it holds is given back."""
        if request_id in self.cache.live:
            self.cache.free_request(request_id)

    # -- the step ------------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request_id!r}: an entry without tokens")
            for t in e.tokens:
                if not 0 <= int(t) < self.model.vocab_size:
                    raise StepError(f"request {e.request_id!r}: token id {t} is outside the vocabulary of {self.model.vocab_size}")
            if self.length(e.request_id) + n > self.max_positions:
                raise StepError(f"request {e.request_id!r}: context length of {self.max_positions} exceeded")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"request {e.request_id!r}: wanted place {w} is not among its {n} tokens")
        new = sum(1 for e in entries if e.request_id not in self.cache.live)
        if len(self.cache.live) + new > self.options.max_requests:
            raise StepError(f"more than {self.options.max_requests} live requests")

    def _fill_batch(self, buf: np.ndarray, layout: StepLayout, entries: Sequence[StepEntry], caches) -> List[int]:
        """Write the step's metadata into `buf` (int32, `layout.total` values); returns the histories."""
        history = [rc.length for rc in caches]
        buf[:] = 0
        tok, pos, rreq = layout.section(buf, 0), layout.section(buf, 1), layout.section(buf, 2)
        for r, e in enumerate(entries):
            a, n = layout.starts[r], layout.counts[r]
            tok[a:a + n] = np.asarray(e.tokens, dtype=np.int64)
            pos[a:a + n] = np.arange(history[r], history[r] + n)
            rreq[a:a + n] = r
        layout.section(buf, 3)[:] = layout.starts
        layout.section(buf, 4)[:] = layout.counts
        layout.section(buf, 5)[:] = history
        layout.section(buf, 6)[:] = [rc.state_slot for rc in caches]
        lr, k = layout.section(buf, 7), 0
        for r, e in enumerate(entries):
            for w in e.want:
                lr[k] = layout.starts[r] + int(w)
                k += 1
        for g, grp in enumerate(self.cache.groups):
            ps = grp.page_size
            bt = layout.section(buf, 8 + 2 * g).reshape(layout.requests, layout.max_pages[g])
            sl = layout.section(buf, 9 + 2 * g)
            for r, rc in enumerate(caches):
                pages = rc.tables[g].pages
                bt[r, :len(pages)] = pages
                parr = np.asarray(pages, dtype=np.int64)
                p = np.arange(history[r], history[r] + layout.counts[r])
                a = layout.starts[r]
                sl[a:a + layout.counts[r]] = parr[p // ps] * ps + p % ps
            # A released page (-1) is never addressed: the window keeps queries above it.
        return history

    def _batch_views(self, dev: torch.Tensor, layout: StepLayout, caches, history: Sequence[int],
                     max_context: int) -> StepBatch:
        """The StepBatch whose device tensors are the sections of `dev`."""
        n_req = layout.requests
        groups = [GroupView(layout.section(dev, 8 + 2 * g).view(n_req, layout.max_pages[g]), layout.section(dev, 9 + 2 * g),
                            grp.page_size) for g, grp in enumerate(self.cache.groups)]
        return StepBatch(rows=layout.rows, requests=n_req, token_ids=layout.section(dev, 0),
                         positions=layout.section(dev, 1), row_request=layout.section(dev, 2),
                         row_start=layout.section(dev, 3), row_count=layout.section(dev, 4),
                         history=layout.section(dev, 5), state_slots=layout.section(dev, 6),
                         logit_rows=layout.section(dev, 7), groups=groups, caches=self.cache,
                         host_row_start=list(layout.starts), host_row_count=list(layout.counts),
                         host_history=list(history), host_state_slots=[rc.state_slot for rc in caches],
                         max_row_count=max(layout.counts), max_context=max_context)

    def _build_batch(self, entries: Sequence[StepEntry], caches) -> StepBatch:
        counts = [len(e.tokens) for e in entries]
        n_groups = len(self.cache.groups)
        max_pages = [max(1, max(len(rc.tables[g].pages) for rc in caches)) for g in range(n_groups)]
        layout = StepLayout(counts, sum(len(e.want) for e in entries), max_pages)
        # One int32 buffer for the whole step, one host-to-device copy.
        host = torch.empty(layout.total, dtype=torch.int32, pin_memory=True)
        history = self._fill_batch(host.numpy(), layout, entries, caches)
        dev = host.to(self.device, non_blocking=True)
        self.last_h2d_bytes = host.numel() * 4
        return self._batch_views(dev, layout, caches, history, max(h + c for h, c in zip(history, counts)))

    def _recording_for(self, entries: Sequence[StepEntry], caches):
        """The recording of this step's shape, made now if the shape has been seen often enough; else None."""
        from . import recorded_step
        counts = tuple(len(e.tokens) for e in entries)
        wants = tuple(tuple(int(w) for w in e.want) for e in entries)
        context = max(rc.length + n for rc, n in zip(caches, counts))
        key = (counts, wants, room_for(context, self.max_positions))
        rec = self.step_recordings.get(key)
        if rec is not None:
            self.step_recordings.move_to_end(key)
            return rec
        seen = self._shapes_seen.get(key, 0)
        if seen < self.options.record_after:
            if len(self._shapes_seen) > 4096:
                self._shapes_seen.clear()
            self._shapes_seen[key] = seen + 1
            return None
        rec = recorded_step.StepRecording(self, counts, wants, key[2])
        self.step_recordings[key] = rec
        self._shapes_seen.pop(key, None)
        while len(self.step_recordings) > recorded_step.MAX_STEP_RECORDINGS:
            self.step_recordings.popitem(last=False)
        return rec

    def step(self, entries: Sequence[StepEntry], record: bool = False) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits [wanted, vocab] on the device, in the order of the
        entries and of each entry's `want`, or None when nothing is wanted.

        `record`: the caller expects steps of this shape (rows per request, wanted places) to come again;
        once one has, the step is recorded as a CUDA graph and replayed from then on (recorded_step.py).
        The logits of a replayed step are valid until the next step of the same shape.

        Raises StepError for a batch it refuses, CacheExhausted when the pages do not suffice;
        in both cases no request has changed.
        """
        self._validate(entries)
        created, prepared = [], []
        try:
            caches = []
            for e in entries:
                rc = self.cache.live.get(e.request_id)
                if rc is None:
                    rc = self.cache.new_request(e.request_id)
                    created.append(e.request_id)
                caches.append(rc)
            for e, rc in zip(entries, caches):
                rc.prepare(len(e.tokens))
                prepared.append(rc)
            with torch.cuda.device(self.device):
                recording = self._recording_for(entries, caches) if record and self.model.recordable else None
                if recording is not None:
                    logits = recording.run(self, entries, caches)
                else:
                    batch = self._build_batch(entries, caches)
                    logits = self.model.forward(batch)
        except BaseException:
            for rc in prepared:
                rc.abort()
            for rid in created:
                self.cache.free_request(rid)
            raise
        for rc in caches:
            rc.commit()
        self.steps_run += 1
        return logits
