"""The two ends of a model: token embedding and the logits head."""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from .. import runtime
from ..weights.spec import TensorSpec
from .base import NativeHandle, Part, Precision, StepBatch
from .linear import Linear, bare_step


class TokenEmbedding(Part):
    """x[r, :] = table[ids[r], :] widened to 32-bit (src/model/arch/blocks.hpp:95-97)."""

    def __init__(self, vocab: int, hidden: int):
        self.vocab, self.hidden = int(vocab), int(hidden)
        self.table: Optional[torch.Tensor] = None
        self._native: Optional[NativeHandle] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab, self.hidden), "table")}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.table = tensors["weight"].to(precision.act).contiguous()
        self._native = None

    @property
    def native(self) -> int:
        if self._native is None:
            runtime.need("rowwise")
            self._native = NativeHandle(runtime.lib().llmx_embedding_create(self.table.data_ptr(), runtime.code(self.table.dtype),
                                                                           self.vocab, self.hidden), keep=(self.table,))
        return self._native.handle

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if not (ids.is_cuda and ids.dtype is torch.int32 and ids.is_contiguous()):
            raise runtime.KernelError("embed: ids must be int32 on the device")
        x = torch.empty((ids.numel(), self.hidden), dtype=torch.float32, device=ids.device)
        s = bare_step(ids.device)
        runtime.check(runtime.lib().llmx_embedding_forward(self.native, ctypes.byref(s), ids.data_ptr(), x.data_ptr(), ids.numel()),
                      "embed")
        return x


class LogitsHead(Part):
    """Logits for the rows that want them: gather, norm, product (src/model/arch/blocks.hpp:267-272).

    The product's weight is the model's own `weight` tensor, or, when `tied_to`
    is given, the embedding's table (the reference's alias, src/model/runtime.hpp:46-53).
    """

    def __init__(self, norm: Part, vocab: int, hidden: int, tied_to: Optional[TokenEmbedding] = None):
        self.norm, self.vocab, self.hidden, self.tied_to = norm, int(vocab), int(hidden), tied_to
        self.linear: Optional[Linear] = None
        self._native: Optional[NativeHandle] = None
        self._native_tried = False

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {} if self.tied_to is not None else {"weight": TensorSpec((self.vocab, self.hidden))}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        if self.tied_to is None:
            self.linear = Linear(tensors["weight"], precision)
        self._native, self._native_tried = None, False

    def bind_tied(self) -> None:
        if self.tied_to is not None:
            self.linear = Linear(self.tied_to.table, self.precision)
            self.linear.weight = self.tied_to.table  # the same memory, not a copy
            self._native, self._native_tried = None, False

    @property
    def native(self):
        if not self._native_tried:
            self._native_tried = True
            norm = self.norm.native
            if norm:
                d = self.linear.desc()
                self._native = NativeHandle(runtime.lib().llmx_head_create(norm, ctypes.byref(d)), keep=(self.norm, self.linear.weight))
        return self._native.handle if self._native is not None else None

    def forward(self, x: torch.Tensor, logit_rows: torch.Tensor) -> torch.Tensor:
        h = self.norm.forward(x, row_index=logit_rows)
        return self.linear(h)
