"""How a layer's parts are arranged.  PreNormBlock: x += mixer(norm(x)); x += ffn(norm(x)).

The names of the four parts (the prefixes of their tensors) are arguments, so
the arrangement knows no architecture's tensor names.  When all four parts have a twin in the native runtime
the block has one too and runs as a single native call; with a part written in Python the block walks its parts
here.
"""
from __future__ import annotations

import ctypes
import inspect
from typing import Dict, Optional

import torch

from .. import runtime
from .base import NativeHandle, Part, StepBatch
from .linear import call_struct


def _cleared(part: Part, rows: int, device, step: StepBatch):
    """The buffer `part` wants zeroed before its forward, if it says so."""
    clear = getattr(part, "wants_cleared", None)
    if clear is None:
        return None
    if "step" in inspect.signature(clear).parameters:
        return clear(rows, device, step)
    return clear(rows, device)


class PreNormBlock(Part):
    def __init__(self, mixer_norm: Part, mixer: Part, ffn_norm: Part, ffn: Part,
                 names=("input_layernorm", "self_attn", "post_attention_layernorm", "mlp")):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.names = tuple(names)
        self._native: Optional[NativeHandle] = None
        self._native_tried = False

    def children(self) -> Dict[str, Part]:
        return dict(zip(self.names, (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)))

    def cache_spec(self):
        return self.mixer.cache_spec()

    def load(self, tensors, precision) -> None:
        super().load(tensors, precision)
        self._native, self._native_tried = None, False

    @property
    def native(self):
        if not self._native_tried:
            self._native_tried = True
            handles = [p.native for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)]
            if all(handles):
                self._native = NativeHandle(runtime.lib().llmx_prenorm_block_create(*handles),
                                            keep=(self.mixer_norm, self.mixer, self.ffn_norm, self.ffn))
        return self._native.handle if self._native is not None else None

    def forward(self, x: torch.Tensor, step: StepBatch, cache_entry: Optional[int], write_cache: bool = True) -> None:
        """x: the float32 residual stream [rows, hidden], updated in place."""
        rows = x.shape[0]
        if self.native is not None:
            rt = runtime.lib()
            probe = step.struct_for(self)
            need = rt.llmx_part_workspace(self.native, ctypes.byref(probe), rows, -1 if cache_entry is None else int(cache_entry))
            runtime.bind_missing()
            s = step.struct_for(self, need)
            runtime.check(rt.llmx_block_forward(self.native, ctypes.byref(s), x.data_ptr(), rows,
                                                -1 if cache_entry is None else int(cache_entry), 1 if write_cache else 0), "block")
            return
        # A part may ask for a buffer to be zeroed before it runs; the norm in front of it does that in passing.
        h = self.mixer_norm.forward(x, zero=_cleared(self.mixer, rows, x.device, step))
        self.mixer.forward(h, step, cache_entry, x, write_cache)
        h = self.ffn_norm.forward(x, zero=_cleared(self.ffn, rows, x.device, step))
        self.ffn.forward(h, step, x)
