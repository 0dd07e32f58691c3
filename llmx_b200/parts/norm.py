"""Norms.  RMSNorm: y = x * (rsqrt(mean(x^2) + eps) * w), 32-bit arithmetic.

The weight is the plain `w` (not `1 + w`), as the reference computes this
architecture (src/backends/cpu/cpu_backend.hpp:1437-1459).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from .. import runtime
from ..weights.spec import TensorSpec
from .base import NativeHandle, Part, Precision
from .linear import bare_step


class RMSNorm(Part):
    def __init__(self, width: int, eps: float):
        self.width, self.eps = int(width), float(eps)
        self.weight: Optional[torch.Tensor] = None
        self._native: Optional[NativeHandle] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.width,), "vector", init="one_plus_normal", std=0.01)}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.weight = tensors["weight"].to(torch.float32).contiguous()
        self._native = None

    @property
    def native(self) -> int:
        if self._native is None:
            runtime.need("rowwise")
            self._native = NativeHandle(runtime.lib().llmx_rmsnorm_create(self.weight.data_ptr(), self.width, self.eps,
                                                                         runtime.code(self.precision.act)), keep=(self.weight,))
        return self._native.handle

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                row_index: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                zero: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`zero`: a float32 buffer the part that follows wants cleared; the norm's launch clears it on the way."""
        rows = x.shape[0] if row_index is None else row_index.numel()
        if out is None:
            out = torch.empty((rows, self.width), dtype=out_dtype or self.precision.act, device=x.device)
        if not (x.is_cuda and x.dtype is torch.float32 and x.is_contiguous() and x.dim() == 2 and x.shape[1] == self.width
                and out.is_contiguous() and tuple(out.shape) == (rows, self.width)
                and (row_index is not None or x.shape[0] >= rows)
                and (row_index is None or (row_index.dtype is torch.int32 and row_index.is_contiguous()))
                and (zero is None or (zero.dtype is torch.float32 and zero.numel() % 4 == 0 and zero.is_contiguous()))):
            raise runtime.KernelError("rmsnorm: float32 rows of the norm's width, an output of as many rows, int32 row_index")
        s = bare_step(x.device)
        runtime.check(runtime.lib().llmx_norm_forward(self.native, ctypes.byref(s), x.data_ptr(), out.data_ptr(), runtime.code(out.dtype),
                                                      runtime.ptr(row_index), rows, runtime.ptr(zero),
                                                      0 if zero is None else zero.numel()), "rmsnorm")
        return out
