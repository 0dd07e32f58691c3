"""A weight matrix [out, in] and its product with the rows of a step.

`Linear` is the one place that decides which matrix-product kernel runs:
on the float32 path the plain CUDA-core product; on the bfloat16 path the
tcgen05 tensor-core product, or the plain one when the input width is not a
multiple of 8 elements (a TMA descriptor needs row strides that are multiples
of 16 bytes).  The choice depends on the weight's shape and the path alone,
never on the batch, so a row's result does not depend on what it was batched
with.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Precision


class Linear:
    def __init__(self, weight: torch.Tensor, precision: Precision):
        # A weight stored in 32-bit is rounded once for the bfloat16 path; a bfloat16 weight
        # is widened exactly for the float32 path.
        self.weight = weight.to(precision.act).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.precision = precision
        self.tensor_core = precision.act is torch.bfloat16 and self.in_features % 8 == 0
        self._tc = None
        self._head_maps = {}

    def __call__(self, a: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                 cleared: bool = False) -> torch.Tensor:
        """out (+)= a @ W.T; a [rows, in] of the path's activation type; out float32 [rows, out].
        `cleared`: `out` already holds zeros (see `output_to_clear`)."""
        if out is None:
            if accumulate:
                raise ValueError("accumulate needs an output to add to")
            out = torch.empty((a.shape[0], self.out_features), dtype=torch.float32, device=a.device)
        if self.tensor_core:
            from .. import ops_tc
            if self._tc is None:
                self._tc = ops_tc.WeightMap(self.weight)
            return ops_tc.gemm_tc(a, self.weight, out, accumulate or cleared and self.adds_pieces(a.shape[0]),
                                  wmap=self._tc)
        return ops.gemm_plain(a, self.weight, out, accumulate)

    def adds_pieces(self, rows: int) -> bool:
        """Whether the product for this many rows adds its pieces into the output with atomics, which then
        must start from zeros when the product is to be stored."""
        if not self.tensor_core:
            return False
        from .. import ops_tc
        return ops_tc.adds_pieces(rows, self.out_features, self.in_features)

    def output_to_clear(self, rows: int, device) -> Optional[torch.Tensor]:
        """A fresh output for `rows` rows if the product wants it cleared by whoever runs before it
        (then pass it back with `cleared=True`), else None."""
        if not self.adds_pieces(rows) or (rows * self.out_features) % 4:
            return None
        return torch.empty((rows, self.out_features), dtype=torch.float32, device=device)

    def gated(self, a: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out = silu(a @ Wg.T) * (a @ Wu.T) for a weight that stacks gate rows on up rows, in one kernel
        (tensor-core path only; the caller checks `fused_gate`)."""
        from .. import ops_tc
        if self._tc is None:
            self._tc = ops_tc.WeightMap(self.weight)
        return ops_tc.gemm_tc_swiglu(a, self.weight, out, wmap=self._tc)

    def fused_gate(self, rows: int) -> bool:
        """Whether the gated form runs for this many rows: with few rows the product is spread over the
        SMs by k ranges, whose partial sums cannot pass through the activation."""
        from .. import ops_tc
        return self.tensor_core and rows > ops_tc.STREAM_K_MAX_ROWS

    def heads(self, a: torch.Tensor, tile: int, heads: int, kv_heads: int, q_weight, k_weight, eps: float, cos, sin,
              positions: torch.Tensor, slots: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor) -> None:
        """The q/k/v product of heads of 128 finished in its epilogue (see ops_tc.gemm_tc_heads; tensor-core path
        only): `tile` weight rows a tile, as `ops_tc.heads_tile` chose."""
        from .. import ops_tc
        wmap = self._head_maps.get(tile)
        if wmap is None:
            wmap = self._head_maps[tile] = ops_tc.WeightMap(self.weight, tile, heads=True)
        ops_tc.gemm_tc_heads(a, wmap, heads, kv_heads, q_weight, k_weight, eps, cos, sin, positions, slots, q_out, cache)
