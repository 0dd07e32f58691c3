"""Feed-forward parts.  GatedMLP: residual += (act(h Wg^T) * (h Wu^T)) Wd^T.

With act = silu this is the SwiGLU block (src/model/arch/blocks.hpp:101-106):
silu(g) = g / (1 + exp(-g)) in 32-bit.  Gate and up weights are stacked by rows
so one product gives both.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import Part, Precision, StepBatch
from .linear import Linear


class GatedMLP(Part):
    def __init__(self, hidden: int, intermediate: int, activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"activation {activation!r} has no kernel here (silu)")
        self.hidden, self.intermediate, self.activation = int(hidden), int(intermediate), activation

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

    def wants_cleared(self, rows: int, device):
        """A buffer this part wants zeroed before `forward` (the norm before it clears it in passing)."""
        self._gu_out = None if self.gate_up.fused_gate(rows) else self.gate_up.output_to_clear(rows, device)
        return self._gu_out

    def forward(self, h: torch.Tensor, step: StepBatch, residual: torch.Tensor) -> None:
        act = torch.empty((h.shape[0], self.intermediate), dtype=self.precision.act, device=h.device)
        out, self._gu_out = getattr(self, "_gu_out", None), None
        if self.gate_up.fused_gate(h.shape[0]):
            self.gate_up.gated(h, act)
        elif out is not None and out.shape[0] == h.shape[0]:
            ops.swiglu(self.gate_up(h, out=out, cleared=True), act)
        else:
            ops.swiglu(self.gate_up(h), act)
        self.down(act, out=residual, accumulate=True)
