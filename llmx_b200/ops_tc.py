"""Python face of the tcgen05 matrix product (csrc/gemm_tc.cu)."""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from . import ops
from .ops import KernelError, _check, _cuda, _fn, _need, _ptr, _stream, register_signature

_i, _p = ctypes.c_int, ctypes.c_void_p
register_signature("gemm_tc", "llmx_gemm_tc_weight_map", [_p, _p, _i, _i])
register_signature("gemm_tc", "llmx_gemm_tc", [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p])
register_signature("gemm_tc", "llmx_gemm_tc_swiglu", [_p, _p, _p, _i, _i, _i, _i, _p, _p])

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


STREAM_K_MAX_ROWS = 64          # at most this many tokens: few tiles, so (tile, k block) units are shared out evenly
STREAM_K_MAX_TILES = 4 * 148    # ... unless the weight alone makes plenty of tiles (the logits head)


def _schedule(m: int, n: int) -> int:
    return 1 if m <= STREAM_K_MAX_ROWS and -(-n // 128) < STREAM_K_MAX_TILES else 0


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
            wmap: Optional[WeightMap] = None, splits: Optional[int] = None, token_tile: int = 0,
            schedule: Optional[int] = None) -> torch.Tensor:
    """out (+)= a @ w.T; a [M, K] bfloat16, w [N, K] bfloat16, out float32 [M, N].

    schedule 0 walks whole tiles (`splits` > 1 cuts K, only with accumulate); schedule 1 (stream-K) shares
    out (tile, k block) units evenly and adds every piece with atomics, zeroing `out` first unless
    accumulating.  By default few tokens take stream-K and many take tiles.
    """
    _cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    _need(a.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and out.dtype is torch.float32,
          "gemm_tc: bfloat16 inputs and a float32 output")
    _need(w.shape[1] == k and tuple(out.shape) == (m, n), "gemm_tc: shapes do not fit")
    _need(k % 8 == 0, "gemm_tc: the input width must be a multiple of 8 (TMA row stride of 16 bytes)")
    wmap = wmap or weight_map(w)
    if schedule is None:
        schedule = _schedule(m, n) if splits is None else 0
    if splits is None:
        splits = 1
    if schedule == 1 and not accumulate:
        out.zero_()
    _check(_fn("gemm_tc", "llmx_gemm_tc")(ctypes.c_void_p(wmap.address), _ptr(a), _ptr(out), m, n, k,
                                          1 if accumulate else 0, splits, token_tile, schedule,
                                          _ptr(error_word(a.device)), _stream()), "gemm_tc")
    return out


def gemm_tc_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, wmap: Optional[WeightMap] = None,
                   token_tile: int = 0) -> torch.Tensor:
    """out = silu(a @ w[:F].T) * (a @ w[F:].T) as bfloat16 [M, F]; w [2F, K] holds the gate rows, then the up rows."""
    _cuda(a, w, out)
    m, k = a.shape
    f = w.shape[0] // 2
    _need(a.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and out.dtype is torch.bfloat16,
          "gemm_tc_swiglu: bfloat16 inputs and output")
    _need(w.shape[0] == 2 * f and w.shape[1] == k and tuple(out.shape) == (m, f), "gemm_tc_swiglu: shapes do not fit")
    _need(k % 8 == 0, "gemm_tc_swiglu: the input width must be a multiple of 8")
    wmap = wmap or weight_map(w)
    _check(_fn("gemm_tc", "llmx_gemm_tc_swiglu")(ctypes.c_void_p(wmap.address), _ptr(a), _ptr(out), m, f, k,
                                                 token_tile, _ptr(error_word(a.device)), _stream()), "gemm_tc_swiglu")
    return out
