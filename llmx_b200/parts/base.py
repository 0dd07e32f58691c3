"""What every part of a layer is, and what a step hands to it.

A model is put together from parts: a *mixer* (attention here), a
*feed-forward*, *norms*, a *position encoding*, arranged in a *block*.  Each
part takes its sizes and constants as constructor arguments, declares the
tensors it reads by role, and runs on whatever rows a step brings.  No part
knows which model it is in; the architecture's builder names the tensors.

Interfaces (what another part of the same kind must provide):

  Part            tensor_specs() -> {role: TensorSpec};  load(tensors, precision)
  Norm            forward(x_f32[T, E], out=None, row_index=None, out_dtype=None, zero=None) -> act[T, E]
                  (`zero`: a float32 buffer the part after it wants cleared; see PreNormBlock)
  PositionEncoding  prepare(max_positions, device); the tables a mixer's kernel reads
  Mixer           cache_spec() -> KVSpec | StateSpec | None
                  forward(h, step, cache_entry, residual, write_cache) adds its output into `residual`
  FeedForward     forward(h, step, residual) adds its output into `residual`
  Block           parts() and forward(x, step, cache_entry, write_cache)

The residual stream `x` is float32 on every path; `h` (a norm's output and the
input of matrix products) has the path's activation type.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import torch

from ..weights.spec import TensorSpec


@dataclass(frozen=True)
class Precision:
    """A numerical path: what matrix products read and what the cache stores.

    bfloat16: bfloat16 weights, activations into products and cache; 32-bit accumulation.
    float32:  everything 32-bit, products on the CUDA cores with explicit fmaf
              (no reduced-precision matrix mode).
    Softmax, norms, rotation angles and the residual sum are 32-bit on both.
    """
    name: str
    act: torch.dtype

    @staticmethod
    def of(name: str) -> "Precision":
        table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
                 "f32": torch.float32}
        if name not in table:
            raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}")
        t = table[name]
        return Precision("bfloat16" if t is torch.bfloat16 else "float32", t)


class Part:
    """Base of every part: tensors by role, loaded once.

    `recordable`: whether the part's forward only enqueues work on the stream (no host read of device
    data), so that a decode step can be recorded in a CUDA graph.  A part that reads results on the
    host sets it to False and is then always run step by step.
    """
    recordable = True

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor], precision: Precision) -> None:
        self.precision = precision

    def children(self) -> Dict[str, "Part"]:
        """Sub-parts by the name their tensors are prefixed with."""
        return {}

    # -- composition ---------------------------------------------------------
    def all_tensor_specs(self, prefix: str = "") -> Dict[str, TensorSpec]:
        out = {prefix + role: spec for role, spec in self.tensor_specs().items()}
        for name, child in self.children().items():
            out.update(child.all_tensor_specs(f"{prefix}{name}."))
        return out

    def load_all(self, fetch, prefix: str, precision: Precision) -> None:
        """`fetch(name, spec)` returns the stored tensor on the device, or None for an absent optional one."""
        mine = {}
        for role, spec in self.tensor_specs().items():
            t = fetch(prefix + role, spec)
            if t is not None:
                mine[role] = t
        self.load(mine, precision)
        for name, child in self.children().items():
            child.load_all(fetch, f"{prefix}{name}.", precision)

    def prepare(self, max_positions: int, device) -> None:
        """Called once before the first step, after load (tables, workspaces)."""
        for child in self.children().values():
            child.prepare(max_positions, device)

    def all_recordable(self) -> bool:
        return self.recordable and all(c.all_recordable() for c in self.children().values())


@dataclass
class GroupView:
    """One cache group's view of the batch."""
    block_tables: torch.Tensor          # int32 [requests, max_pages]
    slots: torch.Tensor                 # int32 [rows]: page * page_size + offset of each row's position
    page_size: int


@dataclass
class StepBatch:
    """Everything a step's kernels need to know about the batch, built once on the host.

    Rows are the tokens of the step in entry order.  Request r of the batch owns rows
    row_start[r] .. row_start[r] + row_count[r]; its history before the step holds
    `history[r]` tokens, so row i of it sits at position history[r] + i.
    """
    rows: int
    requests: int
    token_ids: torch.Tensor             # int32 [rows]
    positions: torch.Tensor             # int32 [rows]
    row_request: torch.Tensor           # int32 [rows]
    row_start: torch.Tensor             # int32 [requests]
    row_count: torch.Tensor             # int32 [requests]
    history: torch.Tensor               # int32 [requests]
    state_slots: torch.Tensor           # int32 [requests] (-1 when the model has no state)
    logit_rows: torch.Tensor            # int32 [wanted]
    groups: List[GroupView]
    caches: Any                         # the CacheManager (entry_storage)
    host_row_start: List[int] = field(default_factory=list)
    host_row_count: List[int] = field(default_factory=list)
    host_history: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)
    max_row_count: int = 0
    max_context: int = 0
    extras: Dict[str, Any] = field(default_factory=dict)   # per-step scratch shared by kernels (schedules)

    def kv(self, cache_entry: int):
        """(group view, this entry's storage [pages, 2, G, page, D])."""
        gi, storage = self.caches.entry_storage(cache_entry)
        return self.groups[gi], storage

    def state(self, cache_entry: int) -> torch.Tensor:
        """The [slots, *shape] state tensor of a state entry."""
        return self.caches.entry_storage(cache_entry)[1]
