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

The framework's own parts run in the native runtime (csrc/runtime/): each holds a
handle (`native`) to its C++ twin, and a block or a model all of whose parts have
one runs as a single native call.  A part written in Python (a test's toy mixer)
has no handle; the blocks and the model that hold it then walk their parts from
Python, calling each part's `forward`, native or not.

Launch plans.  A part whose kernels need decisions taken on the host from the
step's shape (which requests run which kernel, how the keys are cut, scratch
sizes) says so through `plan_step(shape)`; see `StepShape` and `PartPlan`.  The
engine and the recorders know no part's plan: they ask the model, reserve the
ints, and fill them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import runtime
from ..weights.spec import TensorSpec


@dataclass(frozen=True)
class Precision:
    """A numerical path: what matrix products read and what the cache stores by default.

    bfloat16: bfloat16 weights and activations into products; 32-bit accumulation.
    float32:  everything 32-bit, products on the CUDA cores with explicit fmaf
              (no reduced-precision matrix mode).
    Softmax, norms, rotation angles and the residual sum are 32-bit on both.

    `invariant`: every kernel and schedule is chosen by the part's own sizes alone, never by the step's rows: whole
    product tiles with k in one piece and the plain attention kernel.  A row's logits then do not depend on what it
    was batched with, bit for bit (the reference's rule, src/backends/backend.hpp:141-150), at the price of speed;
    without it the bfloat16 path picks product schedules by the step's total rows and adds partial sums with
    atomics, so a row's last bits move with the batch and from run to run.
    """
    name: str
    act: torch.dtype
    invariant: bool = False

    @staticmethod
    def of(name: str, invariant: bool = False) -> "Precision":
        table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
                 "f32": torch.float32}
        if name not in table:
            raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}")
        t = table[name]
        return Precision("bfloat16" if t is torch.bfloat16 else "float32", t, bool(invariant))

    @property
    def flags(self) -> int:
        return runtime.FLAG_INVARIANT if self.invariant else 0


@dataclass
class StepShape:
    """What a launch plan may depend on.  `counts[r]`: rows request r brings; `histories[r]`: tokens before them.
    `room` > 0: the step is recorded and replayed; every decision that shapes a launch (grids, scratch sizes, the
    plan's length) must then follow `counts` and `room` alone (`histories` is None), and `PartPlan.fill` writes what
    follows the histories of the run at hand.  `typical_context` (with room): the context the step that caused the
    recording had, a hint for decisions that are a matter of speed only."""
    counts: Sequence[int]
    histories: Optional[Sequence[int]]
    wants: Sequence[Sequence[int]] = ()
    room: int = 0
    typical_context: int = 0


class PartPlan:
    """A part's launch decisions for one step shape: `ints` values it wants in the step's metadata on the
    device, and `fill(histories, out)` writing them (called every run; `out` is an int32 array of `ints`)."""
    ints = 0

    def fill(self, histories: Sequence[int], out: np.ndarray) -> None:
        pass


class Part:
    """Base of every part: tensors by role, loaded once.

    `recordable`: whether the part's forward only enqueues work on the stream (no host read of device
    data), so that a step can be recorded in a CUDA graph.  A part that reads results on the host sets it
    to False and is then always run step by step.
    `position_streams`: how many position streams of the step the part reads (see StepBatch.positions).
    """
    recordable = True
    position_streams = 1

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor], precision: Precision) -> None:
        self.precision = precision

    def children(self) -> Dict[str, "Part"]:
        """Sub-parts by the name their tensors are prefixed with."""
        return {}

    @property
    def native(self):
        """The part's handle in the native runtime, or None for a part that runs in Python."""
        return None

    def plan_step(self, shape: StepShape) -> Optional[PartPlan]:
        """The part's launch plan for steps of this shape, or None when it needs none.  During `forward` the
        part finds its ints through `step.plan_ints(self)`."""
        return None

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

    def all_parts(self):
        yield self
        for c in self.children().values():
            yield from c.all_parts()


class NativeHandle:
    """Owns one `llmx_part` (destroyed with the Python object that holds it)."""

    def __init__(self, handle: int, keep=()):
        if not handle:
            raise runtime.KernelError(runtime.last_error())
        self.handle = handle
        self.keep = keep              # tensors and handles the native part points into

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h and runtime is not None and runtime._lib is not None:
            runtime._lib.llmx_part_destroy(h)


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

    `position_streams` [streams, rows]: the rows' positions, one stream for most models (stream 0: the position in
    the request); a position encoding with several axes reads the others (`StepEntry.positions`).
    `struct`: the same as an `llmx_step` for the native runtime.
    """
    rows: int
    requests: int
    token_ids: torch.Tensor             # int32 [rows]
    positions: torch.Tensor             # int32 [rows]: stream 0
    row_request: torch.Tensor           # int32 [rows]
    row_start: torch.Tensor             # int32 [requests]
    row_count: torch.Tensor             # int32 [requests]
    history: torch.Tensor               # int32 [requests]
    state_slots: torch.Tensor           # int32 [requests]: the slot each request's state lies in (-1 when the model has none)
    logit_rows: torch.Tensor            # int32 [wanted]
    groups: List[GroupView]
    caches: Any                         # the CacheManager (entry_storage)
    host_row_start: List[int] = field(default_factory=list)
    host_row_count: List[int] = field(default_factory=list)
    host_history: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)
    state_slots_out: Optional[torch.Tensor] = None         # int32 [requests]: the slot the step writes each request's
    #                                                        state to (a request's spare; the two swap when the step is
    #                                                        committed, so a failed step leaves the state as it was)
    host_state_slots_out: List[int] = field(default_factory=list)
    max_row_count: int = 0
    max_context: int = 0
    extras: Dict[str, Any] = field(default_factory=dict)   # per-step scratch shared by Python parts
    position_streams: Optional[torch.Tensor] = None        # int32 [streams, rows]
    struct: Any = None                  # runtime.StepStruct
    plan: Any = None                    # the ModelPlan of this step (models/model.py)
    room: int = 0                       # > 0 inside a recording
    _keep: List[Any] = field(default_factory=list)

    def kv(self, cache_entry: int):
        """(group view, this entry's storage [pages, 2, G, page, D])."""
        gi, storage = self.caches.entry_storage(cache_entry)
        return self.groups[gi], storage

    def state(self, cache_entry: int) -> torch.Tensor:
        """The [slots, *shape] state tensor of a state entry."""
        return self.caches.entry_storage(cache_entry)[1]

    def plan_ints(self, part) -> Optional[torch.Tensor]:
        """The device view of the ints `part.plan_step` asked for, or None."""
        return self.plan.device_ints(part) if self.plan is not None else None

    def struct_for(self, part, workspace_bytes: int = 0):
        """A copy of the step's `llmx_step` for one native part called from Python: its own plan and a workspace."""
        s = runtime.StepStruct.from_buffer_copy(self.struct)
        if self.plan is not None:
            handle, offset = self.plan.native_plan(part)
            s.plan, s.plan_offset = handle, offset
        if workspace_bytes:
            ws = torch.empty(int(workspace_bytes), dtype=torch.uint8, device=self.token_ids.device)
            self._keep.append(ws)
            s.workspace, s.workspace_bytes = ws.data_ptr(), int(workspace_bytes)
        s.stream = runtime.current_stream()
        return s
