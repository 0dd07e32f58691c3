"""The attention mixer: grouped-query attention over the paged cache.

For the rows of a step (src/model/arch/qwen3.hpp:272-295):
    q, k, v = h Wq^T, h Wk^T, h Wv^T            (one product over the stacked weight)
    q, k    = RMSNorm per head (optional), then rotated by position (optional)
    k, v   -> the row's cache slot
    o       = softmax(q K^T / sqrt(D)) V over the request's keys lo..p, causal,
              lo = 0 or p - window + 1; query head h reads kv head h // (H / G)
    residual += o Wo^T
Sizes (heads, kv heads, head width, window), whether q/k are normed, and the
position encoding are constructor arguments.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import ops
from ..cache.manager import KVSpec
from ..weights.spec import TensorSpec
from .base import Part, Precision, StepBatch
from .linear import Linear


class Attention(Part):
    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, position_encoding: Part,
                 qk_norm_eps: Optional[float] = None, window: Optional[int] = None,
                 scale: Optional[float] = None):
        if heads % kv_heads:
            raise ValueError("head count must be divisible by KV head count")
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        self.position_encoding = position_encoding
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.q_width, self.kv_width = self.heads * self.head_dim, self.kv_heads * self.head_dim

    def children(self):
        return {}

    def cache_spec(self):
        return KVSpec(self.kv_heads, self.head_dim, self.window)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {
            "q_proj.weight": TensorSpec((self.q_width, self.hidden)),
            "k_proj.weight": TensorSpec((self.kv_width, self.hidden)),
            "v_proj.weight": TensorSpec((self.kv_width, self.hidden)),
            "o_proj.weight": TensorSpec((self.hidden, self.q_width)),
        }
        if self.qk_norm_eps is not None:
            specs["q_norm.weight"] = TensorSpec((self.head_dim,), "vector", init="one_plus_normal", std=0.01)
            specs["k_norm.weight"] = TensorSpec((self.head_dim,), "vector", init="one_plus_normal", std=0.01)
        return specs

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        # One product for q, k and v: the weights stacked by rows.
        stacked = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0)
        self.qkv = Linear(stacked, precision)
        self.o = Linear(tensors["o_proj.weight"], precision)
        self.q_norm = self.k_norm = None
        if self.qk_norm_eps is not None:
            self.q_norm = tensors["q_norm.weight"].to(torch.float32).contiguous()
            self.k_norm = tensors["k_norm.weight"].to(torch.float32).contiguous()

    def prepare(self, max_positions: int, device) -> None:
        self.position_encoding.prepare(max_positions, device)

    def wants_cleared(self, rows: int, device) -> Optional[torch.Tensor]:
        """A buffer this mixer wants zeroed before `forward` (the norm before it clears it in passing)."""
        from .attention_dispatch import heads_tile
        if heads_tile(self.qkv, rows, self.heads, self.kv_heads, self.head_dim, self.position_encoding.cos):
            self._qkv_out = None        # the product finishes its heads itself: no float32 output to clear
        else:
            self._qkv_out = self.qkv.output_to_clear(rows, device)
        return self._qkv_out

    def forward(self, h: torch.Tensor, step: StepBatch, cache_entry: int, residual: torch.Tensor,
                write_cache: bool = True) -> None:
        rows = h.shape[0]
        group, cache = step.kv(cache_entry)
        out, self._qkv_out = getattr(self, "_qkv_out", None), None
        pe = self.position_encoding
        slots = group.slots
        if not write_cache:
            # A layer that reads another layer's cache computes its queries only.
            key = ("no_write_slots", id(group))
            if key not in step.extras:
                step.extras[key] = torch.full_like(group.slots, -1)
            slots = step.extras[key]
        o = torch.empty((rows, self.q_width), dtype=self.precision.act, device=h.device)
        from .attention_dispatch import decode_from_qkv, heads_from_product, heads_tile, paged_attention
        tile = heads_tile(self.qkv, rows, self.heads, self.kv_heads, self.head_dim, pe.cos)
        q = torch.empty_like(o) if tile else None
        if tile and heads_from_product(self.qkv, h, tile, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, pe.cos,
                                       pe.sin, slots, q, cache, step, self.heads, self.kv_heads):
            # Many rows: the product normed, rotated and stored its heads in its own epilogue.
            paged_attention(q, cache, o, step, group, self.heads, self.kv_heads, self.head_dim, self.window, self.scale)
            self.o(o, out=residual, accumulate=True)
            return
        qkv = self.qkv(h, out=out, cleared=out is not None) if out is not None and out.shape[0] == rows else self.qkv(h)
        # A step of decoding rows only: the attention kernel makes its queries and new keys itself.
        if not decode_from_qkv(qkv, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, pe.cos, pe.sin, slots, cache, o,
                               step, group, self.heads, self.kv_heads, self.head_dim, self.window, self.scale):
            q = torch.empty_like(o)
            ops.head_norm_rope_kv(qkv, self.heads, self.kv_heads, self.head_dim, self.q_norm, self.k_norm,
                                  self.qk_norm_eps or 0.0, pe.cos, pe.sin, step.positions, slots, q, cache)
            paged_attention(q, cache, o, step, group, self.heads, self.kv_heads, self.head_dim, self.window, self.scale)
        self.o(o, out=residual, accumulate=True)
