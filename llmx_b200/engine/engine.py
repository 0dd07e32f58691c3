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
from ..parts.base import Precision, StepBatch, StepShape
from ..registry import architecture_of, config_from_dir
from ..weights.safetensors import TensorDirectory
from . import batch as batching
from .batch import StepLayout


class StepError(ValueError):
    """A batch the step refuses before any work."""


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places whose logits are wanted."""
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    positions: Optional[Sequence[Sequence[int]]] = None   # the tokens' positions in the streams beyond the first
    #                                                       (one list a stream; for position encodings with several
    #                                                       axes; the first stream is always the place in the request)


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"
    kv_dtype: Optional[str] = None   # the cache's element type, "bfloat16" or "float32" (default: the path's).  The
    #                                  reference's cache types are its own options too (ModelOptions.kv_k / kv_v,
    #                                  src/model/runtime.hpp:80-84): bfloat16 products over a float32 cache separate the
    #                                  products' rounding from the cache's; a cache the tiled kernels do not take
    #                                  (anything but bfloat16) runs the plain attention kernel
    kv_tokens: int = 8192            # tokens the cache pool is made for
    window_kv_tokens: Optional[int] = None   # ... the pools of layer groups that keep only a window (default: as many)
    page_size: int = 16
    invariant: bool = False          # kernels and schedules chosen by sizes alone, never by the batch (parts.base.Precision)
    seed: int = 0                    # of the random weights `from_config` makes when it is given none
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


ROOM_STEP = 2048           # a recording's room for context is a multiple of this


def room_for(context: int, max_positions: int) -> int:
    """Tokens of context a recorded step at `context` tokens has room for: at least one `ROOM_STEP`
    ahead, so that recordings change rarely."""
    return min((context // ROOM_STEP + 2) * ROOM_STEP, max(max_positions, 1))


class Engine:
    def __init__(self, model, options: EngineOptions):
        """`model` must be loaded (`Model.load`) on `options.device` in `options.dtype`."""
        if not torch.cuda.is_available():
            raise RuntimeError("llmx_b200 runs on a CUDA device; none is available (there is no CPU path)")
        self.model = model
        self.options = options
        self.device = torch.device(options.device)
        self.precision = Precision.of(options.dtype, options.invariant)
        if model.precision is None or model.precision.act is not self.precision.act:
            raise ValueError("the model was not loaded in the engine's dtype")
        self.max_positions = model.max_positions
        kv_dtype = Precision.of(options.kv_dtype).act if options.kv_dtype else self.precision.act
        specs = model.cache_entry_specs()
        self.cache = CacheManager(specs, options.page_size, options.kv_tokens, options.max_requests, kv_dtype=kv_dtype,
                                  device=self.device, window_kv_tokens=options.window_kv_tokens)
        # Position tables reach as far as a request can: the pool's size where every request's keys all lie in it,
        # the model's context where some group keeps a window only, or nothing but fixed-size state.
        bounded = bool(self.cache.groups) and any(g.spec.window is None for g in self.cache.groups)
        model.prepare(min(self.max_positions, max(options.kv_tokens, 1)) if bounded else self.max_positions, self.device)
        self.position_streams = model.position_streams
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
        self._pinned_ring = [(None, None)] * 4
        self._pinned_at = 0

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
            model.load(source, torch.device(options.device), Precision.of(options.dtype, options.invariant), where=model_dir)
        source.close()
        return cls(model, options)

    @classmethod
    def from_config(cls, config, seed: Optional[int] = None, options: Optional[EngineOptions] = None) -> "Engine":
        """A model of `config` with random weights made on the device (no files); `seed` defaults to the options'."""
        from ..weights.random_init import RandomSource
        options = options or EngineOptions()
        seed = options.seed if seed is None else seed
        config = _scaled(config, options)
        entry = architecture_of(config.to_dict())
        model = entry.build(config)
        src = RandomSource(model.tensor_specs(), seed, dtype=torch.bfloat16, device=options.device, skip_optional=True)
        model.load(src, torch.device(options.device), Precision.of(options.dtype, options.invariant), where="random weights")
        return cls(model, options)

    # -- requests ------------------------------------------------------------------
    def length(self, request_id: Hashable) -> int:
        rc = self.cache.live.get(request_id)
        return rc.length if rc else 0

    def end(self, request_id: Hashable) -> None:
        """The request is finished: what it holds is given back."""
        if request_id in self.cache.live:
            self.cache.free_request(request_id)

    def truncate(self, request_id: Hashable, length: int) -> None:
        """Roll a live request back to its first `length` tokens: the keys beyond are forgotten and their pages
        given back, and the next step continues from there (the reference's KVSequence::truncate,
        src/model/kv_cache.hpp:126-130, which its runtime uses to rewind a prompt whose later chunk failed,
        src/model/runtime.hpp:1347-1353).  Refused for a model with fixed-size state and below what a window gave back."""
        rc = self.cache.live.get(request_id)
        if rc is None:
            raise StepError(f"request {request_id!r} is not live")
        rc.truncate(int(length))

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
            ids = np.asarray(e.tokens)
            if ids.dtype.kind not in "iu" or int(ids.min()) < 0 or int(ids.max()) >= self.model.vocab_size:
                bad = next((t for t in e.tokens if not (isinstance(t, (int, np.integer)) and 0 <= int(t) < self.model.vocab_size)), None)
                raise StepError(f"request {e.request_id!r}: token id {bad} is outside the vocabulary of {self.model.vocab_size}")
            if self.length(e.request_id) + n > self.max_positions:
                raise StepError(f"request {e.request_id!r}: context length of {self.max_positions} exceeded")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"request {e.request_id!r}: wanted place {w} is not among its {n} tokens")
            if e.positions is not None and (len(e.positions) != self.position_streams - 1 or any(len(p) != n for p in e.positions)):
                raise StepError(f"request {e.request_id!r}: positions must be {self.position_streams - 1} lists of {n} "
                                "(one for every position stream of the model beyond the first)")
        new = sum(1 for e in entries if e.request_id not in self.cache.live)
        if len(self.cache.live) + new > self.options.max_requests:
            raise StepError(f"more than {self.options.max_requests} live requests")

    def fill_batch(self, buf: np.ndarray, layout: StepLayout, entries: Sequence[StepEntry], caches) -> List[int]:
        """Write the step's metadata into `buf` (int32, `layout.total` values); returns the histories."""
        history = [rc.length for rc in caches]
        pages = [[rc.tables[g].pages for rc in caches] for g in range(len(self.cache.groups))]
        more = [e.positions for e in entries] if self.position_streams > 1 else None
        batching.fill(buf, layout, [e.tokens for e in entries], history, [rc.state_slot for rc in caches],
                      [e.want for e in entries], pages, [g.page_size for g in self.cache.groups], more,
                      [rc.state_slot_out for rc in caches])
        return history

    def batch_views(self, dev: torch.Tensor, layout: StepLayout, caches, history: Sequence[int], max_context: int,
                    plan=None, room: int = 0) -> StepBatch:
        """The StepBatch whose device tensors are the sections of `dev`."""
        return batching.views(dev, layout, self.cache, [g.page_size for g in self.cache.groups], history,
                              [rc.state_slot for rc in caches], max_context, plan, room,
                              [rc.state_slot_out for rc in caches])

    def _pinned(self, ints: int) -> torch.Tensor:
        """A pinned int32 buffer of `ints` values for a step's metadata, from a small ring: a buffer is used again only
        once the copy that read it has finished."""
        ring = self._pinned_ring
        slot = self._pinned_at = (self._pinned_at + 1) % len(ring)
        buf, event = ring[slot]
        if event is not None:
            event.synchronize()
        if buf is None or buf.numel() < ints:
            buf = torch.empty(max(ints, 4096), dtype=torch.int32, pin_memory=True)
        ring[slot] = (buf, None)
        return buf[:ints]

    def _pinned_done(self, view: torch.Tensor) -> None:
        ev = torch.cuda.Event()
        ev.record()
        self._pinned_ring[self._pinned_at] = (self._pinned_ring[self._pinned_at][0], ev)

    def _build_batch(self, entries: Sequence[StepEntry], caches) -> StepBatch:
        counts = [len(e.tokens) for e in entries]
        history = [rc.length for rc in caches]
        n_groups = len(self.cache.groups)
        max_pages = [max(1, max(len(rc.tables[g].pages) for rc in caches)) for g in range(n_groups)]
        # What the model's parts decide from the shape before anything is launched; their ints ride in the same buffer.
        plan = self.model.plan_step(StepShape(counts, history, [tuple(e.want) for e in entries]))
        layout = StepLayout(counts, sum(len(e.want) for e in entries), max_pages, self.position_streams, plan.ints)
        # One int32 buffer for the whole step, one host-to-device copy.
        host = self._pinned(layout.total)
        buf = host.numpy()
        self.fill_batch(buf, layout, entries, caches)
        plan.fill(history, layout.plan(buf))
        dev = host.to(self.device, non_blocking=True)
        self._pinned_done(host)
        self.last_h2d_bytes = host.numel() * 4
        return self.batch_views(dev, layout, caches, history, max(h + c for h, c in zip(history, counts)), plan)

    def _recording_for(self, entries: Sequence[StepEntry], caches):
        """The recording of this step's shape, made now if the shape has been seen often enough; else None."""
        from . import recording as recorded_step
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
        rec = recorded_step.Recording(self, counts, wants, key[2], typical_context=context)
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
                    from .. import runtime
                    runtime.count_launches(recording.graph_launches)
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
