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
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Set

import torch

from ..parts.base import Part, Precision, StepBatch
from ..parts.embedding import LogitsHead, TokenEmbedding
from ..weights.loader import check_tensors, stored
from ..weights.spec import TensorSpec


@dataclass(frozen=True)
class LayerStep:
    block: int                          # index into Model.blocks
    cache_entry: Optional[int] = None   # index of the cache entry the mixer uses (None: the mixer has no cache)
    write_cache: bool = True            # False: read the entry another step wrote


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

    def prepare(self, max_positions: int, device) -> None:
        for _, part in self._parts():
            part.prepare(max_positions, device)

    @property
    def recordable(self) -> bool:
        """Whether a decode step of this model can be recorded and replayed (every part only enqueues work)."""
        return all(part.all_recordable() for _, part in self._parts())

    # -- one step ------------------------------------------------------------------
    def forward(self, step: StepBatch) -> Optional[torch.Tensor]:
        """Run the step's rows through every layer; logits [wanted, vocab] float32, or None if none is wanted."""
        x = self.embedding.forward(step.token_ids)
        for s in self.order:
            self.blocks[s.block].forward(x, step, s.cache_entry, s.write_cache)
        if step.logit_rows.numel() == 0:
            return None
        return self.head.forward(x, step.logit_rows)
