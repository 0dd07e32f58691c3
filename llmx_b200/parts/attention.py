"""The attention mixer: grouped-query attention over the paged cache.

For the rows of a step (src/model/arch/qwen3.hpp:272-295):
    q, k, v = h Wq^T, h Wk^T, h Wv^T            (one product over the stacked weight)
    q, k    = RMSNorm per head (optional), then rotated by position (optional)
    k, v   -> the row's cache slot
    o       = softmax(q K^T / sqrt(D)) V over the request's keys lo..p, causal,
              lo = 0 or p - window + 1; query head h reads kv head h // (H / G)
    residual += o Wo^T
Sizes (heads, kv heads, head width, window), whether q/k are normed, and the
position encoding are constructor arguments.  The forward pass and the choice of kernels are the native
runtime's (`Attention` in csrc/runtime/runtime.cpp); this class declares the tensors, stacks the weights and
hands the runtime their addresses.
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, Optional

import numpy as np
import torch

from .. import runtime
from ..cache.manager import KVSpec
from ..weights.spec import TensorSpec
from .base import NativeHandle, Part, PartPlan, Precision, StepBatch, StepShape
from .linear import Linear, call_struct


class NativePlan(PartPlan):
    """The runtime's launch plan of a native model or of native parts (`llmx_plan_*`)."""

    def __init__(self, model_handle, part_handles, shape: StepShape):
        self.plan = runtime.Plan(model_handle, list(part_handles), list(shape.counts),
                                 None if shape.histories is None else list(shape.histories), shape.room, shape.typical_context)
        self.ints = self.plan.ints

    def fill(self, histories, out: np.ndarray) -> None:
        self.plan.fill(list(histories), out)


class Attention(Part):
    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, position_encoding: Part,
                 qk_norm_eps: Optional[float] = None, window: Optional[int] = None,
                 scale: Optional[float] = None, position_stream: int = 0):
        if heads % kv_heads:
            raise ValueError("head count must be divisible by KV head count")
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        self.position_encoding = position_encoding
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.q_width, self.kv_width = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.position_stream = int(position_stream)
        self.position_streams = self.position_stream + 1
        self._native: Optional[NativeHandle] = None

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
        self._native = None

    def prepare(self, max_positions: int, device) -> None:
        self.position_encoding.prepare(max_positions, device)
        if self._native is not None:
            self._set_tables()

    def _tables(self):
        pe = self.position_encoding
        cos, sin = getattr(pe, "cos", None), getattr(pe, "sin", None)
        if cos is None:
            return None, None, 0, 0
        if not (cos.dtype is torch.float32 and sin is not None and cos.shape == sin.shape and cos.dim() == 2
                and cos.is_contiguous() and sin.is_contiguous() and 2 * cos.shape[1] <= self.head_dim):
            raise runtime.KernelError("attention: cos and sin tables must be float32 [positions, rot_dim / 2], rot_dim at most the head width")
        return cos, sin, cos.shape[1], cos.shape[0]

    def _set_tables(self) -> None:
        cos, sin, half, n = self._tables()
        runtime.check(runtime.lib().llmx_attention_set_tables(self._native.handle, runtime.ptr(cos), runtime.ptr(sin), half, n),
                      "attention tables")
        self._native.keep = (self.qkv.weight, self.o.weight, self.q_norm, self.k_norm, cos, sin)

    @property
    def native(self) -> int:
        if self._native is None:
            runtime.need("rowwise")
            tiled = self.precision.act is torch.bfloat16 and not self.precision.invariant and \
                runtime.tiled_attention(self.heads, self.kv_heads, self.head_dim, 16)
            if tiled:
                runtime.need("attention_decode")      # its launch plans ask the device which clusters fit
            cos, sin, half, n = self._tables()
            d = runtime.AttentionDesc(self.hidden, self.heads, self.kv_heads, self.head_dim, int(self.window or 0), self.scale,
                                      float(self.qk_norm_eps or 0.0), runtime.ptr(self.q_norm), runtime.ptr(self.k_norm),
                                      runtime.ptr(cos), runtime.ptr(sin), half, n, self.position_stream, self.qkv.desc(),
                                      self.o.desc(), self.precision.flags)
            self._native = NativeHandle(runtime.lib().llmx_attention_create(ctypes.byref(d)),
                                        keep=(self.qkv.weight, self.o.weight, self.q_norm, self.k_norm, cos, sin))
        return self._native.handle

    native_planned = True       # its launch plan is the runtime's: the model gathers such parts into one native plan

    def wants_cleared(self, rows: int, device, step: Optional[StepBatch] = None) -> Optional[torch.Tensor]:
        """A float32 buffer this mixer wants zeroed before `forward` (the norm before it clears it in passing)."""
        s = step.struct_for(self) if step is not None else None
        n = runtime.lib().llmx_part_wants_cleared(self.native, ctypes.byref(s), rows) if s is not None else 0
        self._cleared = torch.empty(int(n), dtype=torch.float32, device=device) if n else None
        return self._cleared

    def forward(self, h: torch.Tensor, step: StepBatch, cache_entry: int, residual: torch.Tensor,
                write_cache: bool = True) -> None:
        rows = h.shape[0]
        cleared, self._cleared = getattr(self, "_cleared", None), None
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("attention: rows of the path's type and the mixer's width, a float32 residual")
        rt = runtime.lib()
        s, _keep = call_struct(step, self, h.device, lambda p: rt.llmx_part_workspace(self.native, ctypes.byref(p), rows, int(cache_entry)))
        runtime.check(rt.llmx_mixer_forward(self.native, ctypes.byref(s), h.data_ptr(), rows, int(cache_entry), residual.data_ptr(),
                                            1 if write_cache else 0, runtime.ptr(cleared)), "attention")
