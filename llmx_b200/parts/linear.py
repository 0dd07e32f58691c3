"""A weight matrix [out, in] and its product with the rows of a step.

The product runs in the native runtime (`Linear` in csrc/runtime/runtime.cpp), which is the one place that
decides which matrix-product kernel runs: on the float32 path the plain CUDA-core product; on the bfloat16 path
the tcgen05 tensor-core product, or the plain one when the input width is not a multiple of 8 elements (a TMA
descriptor needs row strides that are multiples of 16 bytes).

On the bfloat16 path the schedule (stream-K for few rows, else the token tile and the number of k ranges that
fill the SMs) follows the step's total rows, and pieces are added with float atomics in no fixed order: a row's
last bits depend on what it was batched with and move from run to run.  `Precision.invariant` fixes one
schedule (whole tiles, k in one piece) so that they do not; the float32 path always has one order.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import runtime
from .base import NativeHandle, Precision


def bare_step(device) -> runtime.StepStruct:
    """An `llmx_step` that names only the stream and the devices' shared buffers (for a part run outside a step)."""
    s = runtime.StepStruct()
    s.error_word = runtime.error_word(device).data_ptr()
    s.counters = runtime.counters(device).data_ptr()
    s.stream = runtime.current_stream()
    return s


def call_struct(step, part, device, workspace_of):
    """The `llmx_step` for one native part called from Python, with the workspace `workspace_of(struct)` bytes asks
    for (the dry run that sizes it also names the kernel libraries still to be bound).  `step` may be None for a part
    that needs no cache and no plan.  Returns (struct, what must stay alive until the call is enqueued)."""
    probe = step.struct_for(part) if step is not None else bare_step(device)
    need = int(workspace_of(probe))
    runtime.bind_missing()
    if step is not None:
        return step.struct_for(part, need), None
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
    probe.workspace, probe.workspace_bytes = ws.data_ptr(), need
    return probe, ws


class Linear:
    def __init__(self, weight: torch.Tensor, precision: Precision):
        # A weight stored in 32-bit is rounded once for the bfloat16 path; a bfloat16 weight
        # is widened exactly for the float32 path.
        self.weight = weight.to(precision.act).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.precision = precision
        self.tensor_core = precision.act is torch.bfloat16 and self.in_features % 8 == 0
        self._native: Optional[NativeHandle] = None

    def desc(self) -> runtime.LinearDesc:
        runtime.need("gemm_tc" if self.tensor_core else "gemm_plain")
        return runtime.LinearDesc(self.weight.data_ptr(), runtime.code(self.weight.dtype), self.out_features,
                                  self.in_features, self.precision.flags)

    @property
    def native(self) -> int:
        if self._native is None:
            d = self.desc()
            self._native = NativeHandle(runtime.lib().llmx_linear_create(ctypes.byref(d)), keep=(self.weight,))
        return self._native.handle

    def __call__(self, a: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                 cleared: bool = False) -> torch.Tensor:
        """out (+)= a @ W.T; a [rows, in] of the path's activation type; out float32 [rows, out].
        `cleared`: `out` already holds zeros (see `output_to_clear`)."""
        if out is None:
            if accumulate:
                raise ValueError("accumulate needs an output to add to")
            out = torch.empty((a.shape[0], self.out_features), dtype=torch.float32, device=a.device)
        if not (a.is_cuda and a.is_contiguous() and out.is_contiguous() and a.dtype is self.weight.dtype
                and out.dtype is torch.float32 and a.shape[1] == self.in_features
                and tuple(out.shape) == (a.shape[0], self.out_features)):
            raise runtime.KernelError("linear: rows of the weight's type and input width, a float32 output")
        s = bare_step(a.device)
        runtime.check(runtime.lib().llmx_linear_forward(self.native, ctypes.byref(s), a.data_ptr(), a.shape[0], out.data_ptr(),
                                                        1 if accumulate else 0, 1 if cleared else 0), "linear")
        return out

    def adds_pieces(self, rows: int) -> bool:
        """Whether the product for this many rows adds its pieces into the output with atomics, which then
        must start from zeros when the product is to be stored."""
        return bool(runtime.lib().llmx_linear_adds_pieces(self.native, int(rows)))

    def output_to_clear(self, rows: int, device) -> Optional[torch.Tensor]:
        """A fresh output for `rows` rows if the product wants it cleared by whoever runs before it
        (then pass it back with `cleared=True`), else None."""
        if not self.adds_pieces(rows) or (rows * self.out_features) % 4:
            return None
        return torch.empty((rows, self.out_features), dtype=torch.float32, device=device)
