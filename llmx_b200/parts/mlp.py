"""Feed-forward parts.  GatedMLP: residual += (act(h Wg^T) * (h Wu^T)) Wd^T.

With act = silu this is the SwiGLU block (src/model/arch/blocks.hpp:101-106):
silu(g) = g / (1 + exp(-g)) in 32-bit.  Gate and up weights are stacked by rows
so one product gives both.  The forward pass is the native runtime's (`GatedMlp` in csrc/runtime/runtime.cpp).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from .. import runtime
from ..weights.spec import TensorSpec
from .base import NativeHandle, Part, Precision, StepBatch
from .linear import Linear, call_struct


class GatedMLP(Part):
    def __init__(self, hidden: int, intermediate: int, activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"activation {activation!r} has no kernel here (silu)")
        self.hidden, self.intermediate, self.activation = int(hidden), int(intermediate), activation
        self._native: Optional[NativeHandle] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {
            "gate_proj.weight": TensorSpec((self.intermediate, self.hidden)),
            "up_proj.weight": TensorSpec((self.intermediate, self.hidden)),
            "down_proj.weight": TensorSpec((self.hidden, self.intermediate)),
        }

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.gate_up = Linear(torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0), precision)
        self.down = Linear(tensors["down_proj.weight"], precision)
        self._native = None

    @property
    def native(self) -> int:
        if self._native is None:
            runtime.need("rowwise")
            d = runtime.MlpDesc(self.hidden, self.intermediate, self.gate_up.desc(), self.down.desc(), self.precision.flags)
            self._native = NativeHandle(runtime.lib().llmx_gated_mlp_create(ctypes.byref(d)),
                                        keep=(self.gate_up.weight, self.down.weight))
        return self._native.handle

    def wants_cleared(self, rows: int, device, step: Optional[StepBatch] = None):
        """A float32 buffer this part wants zeroed before `forward` (the norm before it clears it in passing)."""
        s = step.struct_for(self) if step is not None else None
        n = runtime.lib().llmx_part_wants_cleared(self.native, ctypes.byref(s), rows) if s is not None else 0
        self._cleared = torch.empty(int(n), dtype=torch.float32, device=device) if n else None
        return self._cleared

    def forward(self, h: torch.Tensor, step: StepBatch, residual: torch.Tensor) -> None:
        rows = h.shape[0]
        cleared, self._cleared = getattr(self, "_cleared", None), None
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("feed-forward: rows of the path's type and the part's width, a float32 residual")
        rt = runtime.lib()
        s, _keep = call_struct(step, self, h.device, lambda p: rt.llmx_part_workspace(self.native, ctypes.byref(p), rows, -1))
        runtime.check(rt.llmx_ffn_forward(self.native, ctypes.byref(s), h.data_ptr(), rows, residual.data_ptr(), runtime.ptr(cleared)),
                      "feed-forward")
