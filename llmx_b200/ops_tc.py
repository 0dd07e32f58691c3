"""Python face of the tcgen05 matrix product (csrc/gemm_tc.cu)."""
from __future__ import annotations

import ctypes
import functools
from typing import Dict, Optional, Tuple

import torch

from . import ops
from .ops import KernelError, _check, _cuda, _fn, _need, _ptr, _stream, register_signature

_i, _p = ctypes.c_int, ctypes.c_void_p
register_signature("gemm_tc", "llmx_gemm_tc_weight_map", [_p, _p, _i, _i])
register_signature("gemm_tc", "llmx_gemm_tc", [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p])
register_signature("gemm_tc_pair", "llmx_gemm_tc_pair", [_p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _p])
register_signature("gemm_tc_pair", "llmx_gemm_tc_pair_swiglu", [_p, _p, _p, _i, _i, _i, _p, _p])
register_signature("gemm_tc_pair", "llmx_gemm_tc_pair_heads", [_p, _p, _i, _i, _p, _p, ctypes.c_float, _p, _p, _p, _p, _p, _p,
                                                               _i, _i, _i, _p, _p])
register_signature("gemm_tc", "llmx_gemm_tc_swiglu", [_p, _p, _p, _i, _i, _i, _i, _p, _p])
register_signature("gemm_tc", "llmx_gemm_tc_weight_map_box", [_p, _p, _i, _i, _i])
register_signature("gemm_tc", "llmx_gemm_tc_heads", [_p, _p, _i, _i, _i, _p, _p, ctypes.c_float, _p, _p, _p, _p, _p, _p,
                                                     _i, _i, _i, _p, _p])

from .runtime import check_errors, error_word      # noqa: F401,E402  (the devices' shared error word lives with the runtime)


class WeightMap:
    """The TMA descriptor of a bfloat16 weight [N, K], made once; 64-byte aligned host memory.
    `box_rows`: the rows one copy brings (128: the weight on the instruction's wide side; 128 or 256 with
    `heads=True`: the weight on the narrow side, whole heads a tile)."""

    def __init__(self, weight: torch.Tensor, box_rows: int = 128, heads: bool = False):
        _need(weight.dtype is torch.bfloat16 and weight.dim() == 2 and weight.is_contiguous() and weight.is_cuda,
              "gemm_tc: the weight must be a contiguous bfloat16 CUDA matrix")
        self.weight = weight
        self.box_rows = box_rows
        self._raw = ctypes.create_string_buffer(128 + 64)
        base = ctypes.addressof(self._raw)
        self.address = (base + 63) & ~63
        n, k = weight.shape
        if heads:
            _check(_fn("gemm_tc", "llmx_gemm_tc_weight_map_box")(ctypes.c_void_p(self.address), _ptr(weight), n, k,
                                                                 box_rows), "gemm_tc weight map")
        else:
            _need(box_rows == 128, "gemm_tc: the wide side takes 128 weight rows a tile")
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


STREAM_K_MAX_ROWS = 64          # at most this many tokens: few tiles, so (tile, k block) units are shared out over all blocks

_sm_count = 0


def _sms() -> int:
    global _sm_count
    if not _sm_count:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def _plan(m: int, n: int, k: int, accumulate: bool, sms: int) -> Tuple[int, int, int]:
    """(schedule, token tile, k ranges) for out[m, n] (+)= a[m, k] w[n, k]^T on a device of `sms` SMs: stream-K for few
    tokens, else whole tiles whose token tile and number of k ranges fill the SMs.  The decision is the native
    runtime's (`gemm_plan_compute` in csrc/runtime/runtime.cpp), which the model's forward pass uses."""
    from . import runtime
    return runtime.gemm_plan(m, n, k, bool(accumulate), sms)


def plan(m: int, n: int, k: int, accumulate: bool) -> Tuple[int, int, int]:
    return _plan(m, n, k, bool(accumulate), _sms())


def adds_pieces(m: int, n: int, k: int) -> bool:
    """Whether a stored product of this shape adds its pieces into the output, which then must start as zeros."""
    schedule, _, splits = plan(m, n, k, False)
    return schedule == 1 or splits != 1


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
            wmap: Optional[WeightMap] = None, splits: Optional[int] = None, token_tile: int = 0,
            schedule: Optional[int] = None) -> torch.Tensor:
    """out (+)= a @ w.T; a [M, K] bfloat16, w [N, K] bfloat16, out float32 [M, N].

    schedule 0 walks whole tiles (`splits` > 1 cuts K and adds the pieces with atomics); schedule 1
    (stream-K) shares out (tile, k block) units over all blocks (in two sizes of run, csrc/gemm_tc.cu) and adds every piece with atomics; schedule 2 walks whole
    tiles of 256 weight rows on pairs of SMs (`gemm_tc_pair`; `splits` 0: the tiles of the last, partial round are cut there).  Whenever pieces
    are added, `out` is zeroed first unless accumulating.  By default `plan` chooses: stream-K for few
    tokens, else the kernel, token tile and k ranges that fill the SMs.
    """
    _cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    _need(a.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and out.dtype is torch.float32,
          "gemm_tc: bfloat16 inputs and a float32 output")
    _need(w.shape[1] == k and tuple(out.shape) == (m, n), "gemm_tc: shapes do not fit")
    _need(k % 8 == 0, "gemm_tc: the input width must be a multiple of 8 (TMA row stride of 16 bytes)")
    wmap = wmap or weight_map(w)
    if schedule is None and splits is None and token_tile == 0:
        schedule, token_tile, splits = plan(m, n, k, accumulate)
    if schedule is None:
        schedule = (1 if plan(m, n, k, accumulate)[0] == 1 else 0) if splits is None else 0
    if splits is None:
        splits = 1
    if schedule == 2:
        return gemm_tc_pair(a, w, out, accumulate, wmap, splits, token_tile or 128)
    if (schedule == 1 or splits > 1) and not accumulate:
        out.zero_()
        accumulate = True
    _check(_fn("gemm_tc", "llmx_gemm_tc")(ctypes.c_void_p(wmap.address), _ptr(a), _ptr(out), m, n, k,
                                          1 if accumulate else 0, splits, token_tile, schedule,
                                          _ptr(error_word(a.device)), _stream()), "gemm_tc")
    return out


def gemm_tc_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, wmap: Optional[WeightMap] = None,
                   token_tile: int = 0, pair: bool = False) -> torch.Tensor:
    """out = silu(a @ w[:F].T) * (a @ w[F:].T) as bfloat16 [M, F]; w [2F, K] holds the gate rows, then the up rows.
    `pair`: on pairs of SMs (csrc/gemm_tc_pair.cu), 256 outputs x 128 tokens a pair."""
    _cuda(a, w, out)
    m, k = a.shape
    f = w.shape[0] // 2
    _need(a.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and out.dtype is torch.bfloat16,
          "gemm_tc_swiglu: bfloat16 inputs and output")
    _need(w.shape[0] == 2 * f and w.shape[1] == k and tuple(out.shape) == (m, f), "gemm_tc_swiglu: shapes do not fit")
    _need(k % 8 == 0, "gemm_tc_swiglu: the input width must be a multiple of 8")
    wmap = wmap or weight_map(w)
    if pair:
        _check(_fn("gemm_tc_pair", "llmx_gemm_tc_pair_swiglu")(ctypes.c_void_p(wmap.address), _ptr(a), _ptr(out), m, f, k,
                                                               _ptr(error_word(a.device)), _stream()), "gemm_tc_pair_swiglu")
        return out
    _check(_fn("gemm_tc", "llmx_gemm_tc_swiglu")(ctypes.c_void_p(wmap.address), _ptr(a), _ptr(out), m, f, k,
                                                 token_tile, _ptr(error_word(a.device)), _stream()), "gemm_tc_swiglu")
    return out


def heads_tile(m: int, heads: int, kv_heads: int) -> int:
    """Weight rows per tile (128: one head, 256: two) of the q/k/v product that finishes its heads in the
    epilogue, or 0 when the tokens are few (the runtime's decision, `heads_tile_compute`).  Timed at 32 heads over
    8, width 4,096 (us, product + per-head kernel -> this): 256 tokens 27 -> 21, 512: 38 -> 32, 1,024: 63 -> 52,
    2,048: 100 -> 88, 8,192: 497 -> 342."""
    from . import runtime
    return runtime.heads_tile(m, heads, kv_heads, _sm_count or 0)


def gemm_tc_heads(a: torch.Tensor, wmap: WeightMap, heads: int, kv_heads: int, q_weight: Optional[torch.Tensor],
                  k_weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                  sin: Optional[torch.Tensor], positions: torch.Tensor, slots: torch.Tensor, q_out: torch.Tensor,
                  cache: torch.Tensor, pair: bool = False) -> None:
    """The q/k/v product of a layer with heads of 128, finished in its epilogue: queries and keys normed per head
    and rotated, queries to `q_out` [M, heads * 128], keys and values to their cache slots.

    a [M, K] bfloat16; `wmap` a `WeightMap(w, 128 | 256, heads=True)` of the stacked weight
    [(heads + 2 kv_heads) * 128, K] (`pair`: on pairs of SMs, 256 tokens x two heads a pair, with a map of 128-row
    boxes); cache [pages, 2, kv_heads, page_size, 128] bfloat16; cos/sin float32
    [positions, 64] or None; positions and slots int32 [M] (a negative slot: the row's key and value are not stored).
    """
    _cuda(a, wmap.weight, q_weight, k_weight, cos, sin, positions, slots, q_out, cache)
    m, k = a.shape
    w = wmap.weight
    _need(a.dtype is torch.bfloat16 and a.is_contiguous() and w.shape[1] == k and k % 8 == 0,
          "gemm_tc_heads: bfloat16 rows of the weight's input width (a multiple of 8)")
    _need(w.shape[0] == (heads + 2 * kv_heads) * 128, "gemm_tc_heads: the weight does not hold heads of 128")
    _need(q_out.dtype is torch.bfloat16 and tuple(q_out.shape) == (m, heads * 128) and q_out.is_contiguous(),
          "gemm_tc_heads: q_out shape does not fit")
    _need(cache.dtype is torch.bfloat16 and cache.dim() == 5 and cache.shape[1] == 2 and cache.shape[2] == kv_heads
          and cache.shape[4] == 128 and cache.is_contiguous(), "gemm_tc_heads: cache layout does not fit")
    _need(positions.dtype == torch.int32 and slots.dtype == torch.int32 and positions.numel() >= m
          and slots.numel() >= m, "gemm_tc_heads: positions and slots must be int32 per row")
    if cos is not None:
        _need(sin is not None and cos.shape == sin.shape and cos.dtype == torch.float32 and cos.dim() == 2
              and cos.shape[1] == 64 and cos.is_contiguous() and sin.is_contiguous(),
              "gemm_tc_heads: cos and sin tables [positions, 64]")
    for nw in (q_weight, k_weight):
        _need(nw is None or (nw.dtype == torch.float32 and nw.numel() == 128), "gemm_tc_heads: norm weight")
    if pair:
        _need(wmap.box_rows == 128, "gemm_tc_heads: on pairs of SMs each block loads one head (boxes of 128 rows)")
        _check(_fn("gemm_tc_pair", "llmx_gemm_tc_pair_heads")(
            ctypes.c_void_p(wmap.address), _ptr(a), m, k, _ptr(q_weight), _ptr(k_weight), float(eps),
            _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slots), _ptr(q_out), _ptr(cache), heads, kv_heads,
            cache.shape[3], _ptr(error_word(a.device)), _stream()), "gemm_tc_pair_heads")
        return
    _check(_fn("gemm_tc", "llmx_gemm_tc_heads")(
        ctypes.c_void_p(wmap.address), _ptr(a), m, k, wmap.box_rows, _ptr(q_weight), _ptr(k_weight), float(eps),
        _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slots), _ptr(q_out), _ptr(cache), heads, kv_heads,
        cache.shape[3], _ptr(error_word(a.device)), _stream()), "gemm_tc_heads")


def gemm_tc_pair(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
                 wmap: Optional[WeightMap] = None, splits: int = 1, token_tile: int = 256) -> torch.Tensor:
    """out (+)= a @ w.T on pairs of SMs (csrc/gemm_tc_pair.cu: tcgen05 `cta_group::2`, a tile of 256 weight rows x
    `token_tile` tokens per pair of thread blocks); a [M, K] bfloat16, w [N, K] bfloat16, out float32 [M, N]."""
    _cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    _need(a.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and out.dtype is torch.float32,
          "gemm_tc_pair: bfloat16 inputs and a float32 output")
    _need(w.shape[1] == k and tuple(out.shape) == (m, n) and k % 8 == 0, "gemm_tc_pair: shapes do not fit")
    wmap = wmap or weight_map(w)
    if splits != 1 and not accumulate:      # pieces of a tile meet by addition (splits 0: the last round's tiles are cut)
        out.zero_()
        accumulate = True
    _check(_fn("gemm_tc_pair", "llmx_gemm_tc_pair")(ctypes.c_void_p(wmap.address), _ptr(a), _ptr(out), m, n, k,
                                                    1 if accumulate else 0, splits, token_tile, _ptr(error_word(a.device)),
                                                    _stream()), "gemm_tc_pair")
    return out
