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


def _pad4(n: int) -> int:
    return (n + 3) & ~3


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
        self.last_h2d_bytes = 0

    # -- construction ------------------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir: str, options: Optional[EngineOptions] = None) -> "Engine":
        """Load a folder with config.json and safetensors; the model class is chosen by config.json."""
        options = options or EngineOptions()
        entry, config = config_from_dir(model_dir)
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

    def _build_batch(self, entries: Sequence[StepEntry], caches) -> StepBatch:
        n_req = len(entries)
        counts = [len(e.tokens) for e in entries]
        rows = sum(counts)
        history = [rc.length for rc in caches]
        starts = np.zeros(n_req, dtype=np.int64)
        np.cumsum(counts[:-1], out=starts[1:])
        wanted = sum(len(e.want) for e in entries)
        n_groups = len(self.cache.groups)
        max_pages = [max(1, max(len(rc.tables[g].pages) for rc in caches)) for g in range(n_groups)]

        # One int32 buffer for the whole step: sections padded to 16 bytes, one host-to-device copy.
        sizes = [rows, rows, rows, n_req, n_req, n_req, n_req, wanted]
        for g in range(n_groups):
            sizes += [n_req * max_pages[g], rows]
        offsets, at = [], 0
        for s in sizes:
            offsets.append(at)
            at += _pad4(max(s, 1))
        host = torch.empty(at, dtype=torch.int32, pin_memory=True)
        buf = host.numpy()
        buf[:] = 0

        def sec(i):
            return buf[offsets[i]:offsets[i] + sizes[i]]

        tok, pos, rreq = sec(0), sec(1), sec(2)
        for r, e in enumerate(entries):
            a, n = int(starts[r]), counts[r]
            tok[a:a + n] = np.asarray(e.tokens, dtype=np.int64)
            pos[a:a + n] = np.arange(history[r], history[r] + n)
            rreq[a:a + n] = r
        sec(3)[:] = starts
        sec(4)[:] = counts
        sec(5)[:] = history
        sec(6)[:] = [rc.state_slot for rc in caches]
        lr, k = sec(7), 0
        for r, e in enumerate(entries):
            for w in e.want:
                lr[k] = int(starts[r]) + int(w)
                k += 1
        for g in range(n_groups):
            ps = self.cache.groups[g].page_size
            bt = sec(8 + 2 * g).reshape(n_req, max_pages[g])
            sl = sec(9 + 2 * g)
            for r, rc in enumerate(caches):
                pages = rc.tables[g].pages
                bt[r, :len(pages)] = pages
                parr = np.asarray(pages, dtype=np.int64)
                p = np.arange(history[r], history[r] + counts[r])
                a = int(starts[r])
                sl[a:a + counts[r]] = parr[p // ps] * ps + p % ps
            # A released page (-1) is never addressed: the window keeps queries above it.
        dev = host.to(self.device, non_blocking=True)
        self.last_h2d_bytes = host.numel() * 4

        def dsec(i):
            return dev[offsets[i]:offsets[i] + sizes[i]]

        groups = [GroupView(dsec(8 + 2 * g).view(n_req, max_pages[g]), dsec(9 + 2 * g), self.cache.groups[g].page_size)
                  for g in range(n_groups)]
        return StepBatch(rows=rows, requests=n_req, token_ids=dsec(0), positions=dsec(1), row_request=dsec(2),
                         row_start=dsec(3), row_count=dsec(4), history=dsec(5), state_slots=dsec(6),
                         logit_rows=dsec(7), groups=groups, caches=self.cache,
                         host_row_start=[int(s) for s in starts], host_row_count=counts, host_history=history,
                         host_state_slots=[rc.state_slot for rc in caches],
                         max_row_count=max(counts), max_context=max(h + c for h, c in zip(history, counts)))

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits [wanted, vocab] on the device, in the order of the
        entries and of each entry's `want`, or None when nothing is wanted.

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
