"""Norms.  RMSNorm: y = x * (rsqrt(mean(x^2) + eps) * w), 32-bit arithmetic.

The weight is the plain `w` (not `1 + w`), as the reference computes this
architecture (src/backends/cpu/cpu_backend.hpp:1437-1459).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import Part, Precision


class RMSNorm(Part):
    def __init__(self, width: int, eps: float):
        self.width, self.eps = int(width), float(eps)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.width,), "vector", init="one_plus_normal", std=0.01)}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.weight = tensors["weight"].to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                row_index: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                zero: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`zero`: a float32 buffer the part that follows wants cleared; the norm's launch clears it on the way."""
        rows = x.shape[0] if row_index is None else row_index.numel()
        if out is None:
            out = torch.empty((rows, self.width), dtype=out_dtype or self.precision.act, device=x.device)
        return ops.rmsnorm(x, self.weight, self.eps, out, row_index, zero)
