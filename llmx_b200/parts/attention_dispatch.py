"""Which attention kernel runs for which rows of a step.

The float32 path, and any shape the tiled kernels do not take, runs the plain
kernel (one block per row and head).  On the bfloat16 path requests that bring
one or a few rows run the split-KV decode kernel and requests that bring a
portion of a prompt run the tiled prefill kernel; both read the same pages and
differ only in rounding.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import GroupView, StepBatch


def paged_attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, step: StepBatch, group: GroupView,
                    heads: int, kv_heads: int, head_dim: int, window: Optional[int], scale: float) -> None:
    if q.dtype is torch.bfloat16:
        from .. import ops_attn
        if ops_attn.supported(heads, kv_heads, head_dim, cache.shape[3]):
            ops_attn.paged_attention_bf16(q, cache, out, step, group, heads, kv_heads, head_dim, window, scale)
            return
    ops.attention_plain(q, cache, out, step.row_request, step.positions, group.block_tables, heads, kv_heads,
                        head_dim, window, scale)


def decode_from_qkv(qkv: torch.Tensor, q_weight, k_weight, eps: float, cos, sin, slots: torch.Tensor,
                    cache: torch.Tensor, out: torch.Tensor, step: StepBatch, group: GroupView, heads: int,
                    kv_heads: int, head_dim: int, window: Optional[int], scale: float) -> bool:
    """On the bfloat16 path, when every request of the step brings few rows and the shapes allow it, the decode
    kernel takes the q/k/v product's output as it is (see ops_attn.decode_from_qkv); else False and nothing done."""
    if out.dtype is not torch.bfloat16:
        return False
    from .. import ops_attn
    return ops_attn.decode_from_qkv(qkv, q_weight, k_weight, eps, cos, sin, slots, cache, out, step, group, heads,
                                    kv_heads, head_dim, window, scale)


def heads_tile(linear, rows: int, heads: int, kv_heads: int, head_dim: int, cos) -> int:
    """Weight rows per tile when the q/k/v product can finish its heads itself for this many rows (bfloat16 path,
    heads of 128, rotation of the whole head or none), else 0."""
    if not linear.tensor_core or head_dim != 128 or (cos is not None and cos.shape[1] != 64):
        return 0
    from .. import ops_tc
    return ops_tc.heads_tile(rows, heads, kv_heads)


def heads_from_product(linear, h: torch.Tensor, tile: int, q_weight, k_weight, eps: float, cos, sin,
                       slots: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, step: StepBatch, heads: int,
                       kv_heads: int) -> bool:
    """Run the q/k/v product with the per-head norm, the rotation and the cache write in its epilogue
    (ops_tc.gemm_tc_heads).  False, having done nothing, when the cache is not bfloat16 or the step is one of
    decoding rows only (the decode kernel then takes the product's output itself)."""
    if cache.dtype is not torch.bfloat16 or q.dtype is not torch.bfloat16:
        return False
    from .. import ops_attn
    if not step.extras.get("no_qkv_attention") and ops_attn.decoding_rows_only(step, heads, kv_heads):
        return False
    linear.heads(h, tile, heads, kv_heads, q_weight, k_weight, eps, cos, sin, step.positions, slots, q, cache)
    return True
