"""How a layer's parts are arranged.  PreNormBlock: x += mixer(norm(x)); x += ffn(norm(x)).

The names of the four parts (the prefixes of their tensors) are arguments, so
the arrangement knows no architecture's tensor names.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Part, StepBatch


class PreNormBlock(Part):
    def __init__(self, mixer_norm: Part, mixer: Part, ffn_norm: Part, ffn: Part,
                 names=("input_layernorm", "self_attn", "post_attention_layernorm", "mlp")):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.names = tuple(names)

    def children(self) -> Dict[str, Part]:
        return dict(zip(self.names, (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)))

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, x: torch.Tensor, step: StepBatch, cache_entry: Optional[int], write_cache: bool = True) -> None:
        """x: the float32 residual stream [rows, hidden], updated in place."""
        rows = x.shape[0]
        # A part may ask for a buffer to be zeroed before it runs; the norm in front of it does that in passing.
        clear = getattr(self.mixer, "wants_cleared", None)
        h = self.mixer_norm.forward(x, zero=clear(rows, x.device) if clear else None)
        self.mixer.forward(h, step, cache_entry, x, write_cache)
        clear = getattr(self.ffn, "wants_cleared", None)
        h = self.ffn_norm.forward(x, zero=clear(rows, x.device) if clear else None)
        self.ffn.forward(h, step, x)
