"""A model: an embedding, blocks, the order they run in, and a head.

The order is data: a list of `LayerStep(block, cache_entry, write_cache)`.
It may name a block twice (the same weights run again, on a cache entry of
their own or on a shared one) and may let a block read the cache entry another
block wrote (`write_cache=False`).  Cache entries are numbered by the model;
what each needs (`KVSpec`, `StateSpec` or nothing) is asked of the mixer of the
first step that names it.

`Model` knows no architecture.  An architecture's builder
(`llmx_b200/models/qwen3.py`) constructs the parts from its configuration and
gives the tensor names.
"""
from __future__ import annotations

from dataclasses import dataclass
import ctypes
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple

import numpy as np
import torch

from .. import runtime
from ..parts.base import NativeHandle, Part, PartPlan, Precision, StepBatch, StepShape
from ..parts.embedding import LogitsHead, TokenEmbedding
from ..weights.loader import check_tensors, stored
from ..weights.spec import TensorSpec


@dataclass(frozen=True)
class LayerStep:
    block: int                          # index into Model.blocks
    cache_entry: Optional[int] = None   # index of the cache entry the mixer uses (None: the mixer has no cache)
    write_cache: bool = True            # False: read the entry another step wrote


class ModelPlan:
    """The launch plans of a model's parts for one step shape, laid out one after the other in the step's
    metadata: first the native runtime's (all native parts share one), then those of parts written in Python."""

    def __init__(self, native: Optional[PartPlan], python: List[Tuple[Part, PartPlan]]):
        self.native = native
        self.python = python
        self.offsets: Dict[int, int] = {}
        at = native.ints if native is not None else 0
        for part, plan in python:
            self.offsets[id(part)] = at
            at += (plan.ints + 3) & ~3
        self.ints = at
        self.base = 0                     # where the plan's ints begin in the step's metadata (set by the engine)
        self.device: Optional[torch.Tensor] = None

    def fill(self, histories: Sequence[int], out: np.ndarray) -> None:
        if self.native is not None:
            self.native.fill(histories, out[:self.native.ints])
        for part, plan in self.python:
            at = self.offsets[id(part)]
            plan.fill(histories, out[at:at + plan.ints])

    def device_ints(self, part: Part) -> Optional[torch.Tensor]:
        for p, plan in self.python:
            if p is part:
                at = self.offsets[id(part)]
                return self.device[at:at + plan.ints]
        return None

    def plan_of(self, part: Part) -> Optional[PartPlan]:
        for p, plan in self.python:
            if p is part:
                return plan
        return None

    def native_plan(self, part=None) -> Tuple[Optional[int], int]:
        """(the runtime's plan handle, where its ints begin in the metadata)."""
        if self.native is None:
            return None, 0
        return self.native.plan.handle, self.base


class Model:
    def __init__(self, *, embedding: TokenEmbedding, blocks: Sequence[Part], head: LogitsHead,
                 order: Optional[Sequence[LayerStep]] = None,
                 block_prefix: Callable[[int], str] = lambda i: f"model.layers.{i}.",
                 embedding_prefix: str = "model.embed_tokens.", head_norm_prefix: str = "model.norm.",
                 head_prefix: str = "lm_head.", vocab_size: int, max_positions: int,
                 ignorable: Iterable[str] = (), eos_ids: Sequence[int] = ()):
        self.embedding, self.blocks, self.head = embedding, list(blocks), head
        self.order: List[LayerStep] = list(order) if order is not None else [
            LayerStep(i, i) for i in range(len(self.blocks))]
        self.block_prefix = block_prefix
        self.embedding_prefix, self.head_norm_prefix, self.head_prefix = embedding_prefix, head_norm_prefix, head_prefix
        self.vocab_size, self.max_positions = int(vocab_size), int(max_positions)
        self.ignorable: Set[str] = set(ignorable)
        self.eos_ids = tuple(eos_ids)
        self.precision: Optional[Precision] = None
        self._native: Optional[NativeHandle] = None
        self._native_tried = False
        self._check_order()

    def _check_order(self) -> None:
        writers: Dict[int, int] = {}
        for n, s in enumerate(self.order):
            if not 0 <= s.block < len(self.blocks):
                raise ValueError(f"layer order step {n} names block {s.block}, the model has {len(self.blocks)}")
            spec = self.blocks[s.block].cache_spec()
            if spec is None:
                if s.cache_entry is not None:
                    raise ValueError(f"layer order step {n}: block {s.block} has no cache but an entry is named")
                continue
            if s.cache_entry is None:
                raise ValueError(f"layer order step {n}: block {s.block} needs a cache entry")
            if s.write_cache:
                if s.cache_entry in writers:
                    raise ValueError(f"layer order steps {writers[s.cache_entry]} and {n} both write cache entry {s.cache_entry}")
                writers[s.cache_entry] = n
            elif s.cache_entry not in writers:
                raise ValueError(f"layer order step {n} reads cache entry {s.cache_entry} before any step wrote it")
        entries = sorted({s.cache_entry for s in self.order if s.cache_entry is not None})
        if entries != list(range(len(entries))):
            raise ValueError("cache entries must be numbered 0..n-1 without gaps")

    # -- what the cache manager needs ------------------------------------------
    def cache_entry_specs(self) -> list:
        specs: Dict[int, object] = {}
        for s in self.order:
            if s.cache_entry is None:
                continue
            spec = self.blocks[s.block].cache_spec()
            if s.cache_entry in specs and specs[s.cache_entry] != spec:
                raise ValueError(f"cache entry {s.cache_entry} is used by mixers with different needs")
            specs[s.cache_entry] = spec
        return [specs[i] for i in range(len(specs))]

    # -- tensors -----------------------------------------------------------------
    def _parts(self):
        yield self.embedding_prefix, self.embedding
        for i, b in enumerate(self.blocks):
            yield self.block_prefix(i), b
        yield self.head_norm_prefix, self.head.norm
        yield self.head_prefix, self.head

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for prefix, part in self._parts():
            if part is self.head:
                out.update({prefix + r: s for r, s in part.tensor_specs().items()})
            else:
                out.update(part.all_tensor_specs(prefix))
        return out

    def load(self, source, device, precision: Precision, where: str = "model") -> None:
        """Check `source` against the model's tensors, then give each part its own, on `device`."""
        specs = self.tensor_specs()
        check_tensors(specs, source, where, self.ignorable)
        have = set(source.names())

        def fetch(name: str, spec: TensorSpec):
            if name not in have:
                return None
            return stored(source, name, spec, device)

        for prefix, part in self._parts():
            if part is self.head:
                mine = {r: fetch(prefix + r, s) for r, s in part.tensor_specs().items()}
                part.load(mine, precision)
            else:
                part.load_all(fetch, prefix, precision)
        self.head.bind_tied()
        self.precision = precision
        self._native, self._native_tried = None, False

    def prepare(self, max_positions: int, device) -> None:
        for _, part in self._parts():
            part.prepare(max_positions, device)

    @property
    def recordable(self) -> bool:
        """Whether a decode step of this model can be recorded and replayed (every part only enqueues work)."""
        return all(part.all_recordable() for _, part in self._parts())

    @property
    def position_streams(self) -> int:
        """How many position streams a step must carry for this model's parts."""
        return max((p.position_streams for _, part in self._parts() for p in part.all_parts()), default=1)

    # -- the native twin ---------------------------------------------------------
    @property
    def native(self) -> Optional[int]:
        """The model's handle in the native runtime when every part has one (else None: the layer order is walked
        from Python, each part running its own forward, native or not)."""
        if not self._native_tried:
            self._native_tried = True
            blocks = [b.native for b in self.blocks]
            emb, head = self.embedding.native, self.head.native
            if emb and head and all(blocks):
                arr = (ctypes.c_void_p * len(blocks))(*blocks)
                order = (runtime.LayerStepStruct * len(self.order))(*[
                    runtime.LayerStepStruct(s.block, -1 if s.cache_entry is None else s.cache_entry, 1 if s.write_cache else 0)
                    for s in self.order])
                handle = runtime.lib().llmx_model_create(emb, arr, len(blocks), order, len(self.order), head,
                                                        self.embedding.hidden, self.vocab_size)
                self._native = _ModelHandle(handle, keep=(self.embedding, self.blocks, self.head))
        return self._native.handle if self._native is not None else None

    # -- launch plans ------------------------------------------------------------
    def plan_step(self, shape: StepShape) -> ModelPlan:
        """What the model's parts decide on the host for steps of this shape (see parts/base.py)."""
        from ..parts.attention import NativePlan
        native = None
        if self.native is not None:
            native = NativePlan(self.native, (), shape)
        else:
            handles = [p.native for _, part in self._parts() for p in part.all_parts() if getattr(p, "native_planned", False)]
            if handles:
                native = NativePlan(None, handles, shape)
        if native is not None and native.ints == 0:
            native = None
        python = []
        if self.native is None:
            seen = set()
            for _, part in self._parts():
                for p in part.all_parts():
                    if id(p) in seen or getattr(p, "native_planned", False):
                        continue
                    seen.add(id(p))
                    plan = p.plan_step(shape)
                    if plan is not None and plan.ints:
                        python.append((p, plan))
        return ModelPlan(native, python)

    # -- one step ------------------------------------------------------------------
    def forward(self, step: StepBatch) -> Optional[torch.Tensor]:
        """Run the step's rows through every layer; logits [wanted, vocab] float32, or None if none is wanted."""
        wanted = step.logit_rows.numel()
        if self.native is not None:
            rt = runtime.lib()
            probe = step.struct_for(self)
            need = rt.llmx_model_workspace(self.native, ctypes.byref(probe))
            runtime.bind_missing()
            s = step.struct_for(self, need)
            logits = torch.empty((wanted, self.vocab_size), dtype=torch.float32, device=step.token_ids.device) if wanted else None
            runtime.check(rt.llmx_model_forward(self.native, ctypes.byref(s), runtime.ptr(logits)), "forward")
            return logits
        x = self.embedding.forward(step.token_ids)
        for s in self.order:
            self.blocks[s.block].forward(x, step, s.cache_entry, s.write_cache)
        if wanted == 0:
            return None
        return self.head.forward(x, step.logit_rows)


class _ModelHandle(NativeHandle):
    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h and runtime._lib is not None:
            runtime._lib.llmx_model_destroy(h)
