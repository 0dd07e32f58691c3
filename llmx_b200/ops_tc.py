"""Python face of the tcgen05 matrix product (csrc/gemm_tc.cu)."""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from . import ops
from .ops import KernelError, _check, _cuda, _fn, _need, _ptr, _stream, register_signature

_i, _p = ctypes.c_int, ctypes.c_void_p
register_signature("gemm_tc", "llmx_gemm_tc_weight_map", [_p, _p, _i, _i])
register_signature("gemm_tc", "llmx_gemm_tc", [_p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _p])

_error_words: Dict[int, torch.Tensor] = {}
_ERROR_NAMES = {101: "the TMA producer waited for a free stage", 102: "the MMA issuer waited for a loaded stage",
                103: "the MMA issuer waited for a free accumulator", 104: "the epilogue waited for an accumulator"}


def error_word(device) -> torch.Tensor:
    """The device int a kernel of this module records a failed wait in (one per device)."""
    idx = torch.device(device).index or 0
    w = _error_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _error_words[idx] = w
    return w


def check_errors() -> None:
    """Raise if any tensor-core kernel gave up a wait (synchronises the devices that ran one)."""
    for idx, w in _error_words.items():
        code = int(w.item())
        if code:
            w.zero_()
            raise KernelError(f"tensor-core kernel on device {idx} gave up: {_ERROR_NAMES.get(code, code)}")


class WeightMap:
    """The TMA descriptor of a bfloat16 weight [N, K], made once; 64-byte aligned host memory."""

    def __init__(self, weight: torch.Tensor):
        _need(weight.dtype is torch.bfloat16 and weight.dim() == 2 and weight.is_contiguous() and weight.is_cuda,
              "gemm_tc: the weight must be a contiguous bfloat16 CUDA matrix")
        self.weight = weight
        self._raw = ctypes.create_string_buffer(128 + 64)
        base = ctypes.addressof(self._raw)
        self.address = (base + 63) & ~63
        n, k = weight.shape
        _check(_fn("gemm_tc", "llmx_gemm_tc_weight_map")(ctypes.c_void_p(self.address), _ptr(weight), n, k),
               "gemm_tc weight map")


_maps: Dict[Tuple[int, int, int], WeightMap] = {}


def weight_map(weight: torch.Tensor) -> WeightMap:
    key = (weight.data_ptr(), weight.shape[0], weight.shape[1])
    m = _maps.get(key)
    if m is None or m.weight is not weight:
        m = WeightMap(weight)
        _maps[key] = m
    return m


def _splits(m: int, n: int, k: int, accumulate: bool, sms: int = 148) -> int:
    """K splits for a product whose tiles alone would leave most of the GPU idle."""
    if not accumulate:
        return 1
    tiles = -(-n // 128) * -(-m // 256 if m > 128 else 1)
    if tiles >= sms // 2:
        return 1
    k_blocks = -(-k // 64)
    return max(1, min(sms // tiles, k_blocks // 8, 8))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
            wmap: Optional[WeightMap] = None, splits: Optional[int] = None, token_tile: int = 0) -> torch.Tensor:
    """out (+)= a @ w.T; a [M, K] bfloat16, w [N, K] bfloat16, out float32 [M, N]."""
    _cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    _need(a.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and out.dtype is torch.float32,
          "gemm_tc: bfloat16 inputs and a float32 output")
    _need(w.shape[1] == k and tuple(out.shape) == (m, n), "gemm_tc: shapes do not fit")
    _need(k % 8 == 0, "gemm_tc: the input width must be a multiple of 8 (TMA row stride of 16 bytes)")
    wmap = wmap or weight_map(w)
    if splits is None:
        splits = _splits(m, n, k, accumulate)
    _check(_fn("gemm_tc", "llmx_gemm_tc")(ctypes.c_void_p(wmap.address), _ptr(a), _ptr(out), m, n, k,
                                          1 if accumulate else 0, splits, token_tile,
                                          _ptr(error_word(a.device)), _stream()), "gemm_tc")
    return out
