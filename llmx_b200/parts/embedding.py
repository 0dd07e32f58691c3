"""The two ends of a model: token embedding and the logits head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import Part, Precision, StepBatch
from .linear import Linear


class TokenEmbedding(Part):
    """x[r, :] = table[ids[r], :] widened to 32-bit (src/model/arch/blocks.hpp:95-97)."""

    def __init__(self, vocab: int, hidden: int):
        self.vocab, self.hidden = int(vocab), int(hidden)
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab, self.hidden), "table")}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.table = tensors["weight"].to(precision.act).contiguous()

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        x = torch.empty((ids.numel(), self.hidden), dtype=torch.float32, device=ids.device)
        return ops.embed(self.table, ids, x)


class LogitsHead(Part):
    """Logits for the rows that want them: gather, norm, product (src/model/arch/blocks.hpp:267-272).

    The product's weight is the model's own `weight` tensor, or, when `tied_to`
    is given, the embedding's table (the reference's alias, src/model/runtime.hpp:46-53).
    """

    def __init__(self, norm: Part, vocab: int, hidden: int, tied_to: Optional[TokenEmbedding] = None):
        self.norm, self.vocab, self.hidden, self.tied_to = norm, int(vocab), int(hidden), tied_to
        self.linear: Optional[Linear] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {} if self.tied_to is not None else {"weight": TensorSpec((self.vocab, self.hidden))}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        if self.tied_to is None:
            self.linear = Linear(tensors["weight"], precision)

    def bind_tied(self) -> None:
        if self.tied_to is not None:
            self.linear = Linear(self.tied_to.table, self.precision)
            self.linear.weight = self.tied_to.table  # the same memory, not a copy

    def forward(self, x: torch.Tensor, logit_rows: torch.Tensor) -> torch.Tensor:
        h = self.norm.forward(x, row_index=logit_rows)
        return self.linear(h)
