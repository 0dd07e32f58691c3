"""Python faces of single CUDA kernels.

The model's forward pass calls the kernels from the native runtime (llmx_b200/runtime.py, csrc/runtime/); the
functions here call one kernel each, for tests that hold a kernel to its plain reference and for parts written
in Python.  Every function launches hand-written sm_100a kernels from `csrc/` on the
current CUDA stream and returns at once.  Arguments are torch tensors on one
CUDA device; shapes, types and contiguity are checked here, on the host, before
a launch, so that a kernel is never handed memory it would read out of bounds.
There is no CPU path and no library fallback: without a GPU or a working nvcc
these functions raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_CODE = {torch.float32: F32, torch.bfloat16: BF16}


from .runtime import KernelError      # noqa: E402  (one error type for kernels and runtime)


def _code(t: torch.Tensor) -> int:
    try:
        return _CODE[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not one the kernels take (float32, bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    """The current stream of the current device (the raw handle: this runs before every launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(cond: bool, what: str) -> None:
    if not cond:
        raise KernelError(what)


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None:
            _need(t.is_cuda, "kernel arguments must be CUDA tensors (there is no CPU path)")
            _need(t.is_contiguous(), "kernel arguments must be contiguous")


_ERRORS = {10001: "bad argument", 10002: "shape or type not supported by this kernel",
           10003: "TMA descriptor could not be encoded", 10004: "size beyond the stated maximum"}


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far: by the native runtime (the model's forward pass, replayed
    recordings included) and by the single-kernel functions of this module."""
    from . import runtime
    return _launches + runtime.launches()


def count_launches(n: int) -> None:
    """Adds the kernels a replayed recording launches."""
    global _launches
    _launches += n


def _check(status: int, what: str, launches: int = 1) -> None:
    global _launches
    _launches += launches
    if status != 0:
        why = _ERRORS.get(status, f"CUDA error {status}")
        raise KernelError(f"{what}: {why}")


_i, _f, _p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_SIGNATURES = {
    ("rowwise", "llmx_embed"): [_p, _i, _p, _p, _i, _i, _i, _p],
    ("rowwise", "llmx_rmsnorm"): [_p, _p, _p, _i, _p, _i, _i, _f, _p, ctypes.c_longlong, _p],
    ("rowwise", "llmx_head_norm_rope_kv"): [_p, _i, _i, _i, _p, _p, _f, _p, _p, _i, _p, _p, _p, _i, _p, _i,
                                            _i, _i, _i, _i, _i, _p],
    ("rowwise", "llmx_swiglu"): [_p, _p, _i, _i, _i, _p],
    ("gemm_plain", "llmx_gemm_plain"): [_p, _i, _p, _i, _p, _i, _i, _i, _i, _p],
    ("attention_plain", "llmx_attention_plain"): [_p, _i, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _p],
}
_fns = {}


_timed_calls = None       # while `kernel_times` is open: [(exported function, start event, end event)]


def _fn(lib: str, name: str):
    key = (lib, name)
    f = _fns.get(key)
    if f is None:
        f = getattr(_build.load(lib), name)
        f.argtypes = _SIGNATURES[key]
        f.restype = ctypes.c_int
        _fns[key] = f
    if _timed_calls is None:
        return f

    def timed(*args):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        status = f(*args)
        end.record()
        _timed_calls.append((name, start, end))
        return status
    return timed


class kernel_times:
    """Device time of every kernel call made inside the `with` block, by exported function (the reference's
    `bench --profile`, src/cli/main.cpp:1326-1352): CUDA events around each call on its stream, in the native
    runtime (the model's forward pass) and in this module's single-kernel functions.  For plain
    steps only: a step that replays a recording makes no calls, and events must not be recorded into one.
    The events keep a kernel from starting while the one before drains, so the times are those of kernels alone."""

    def __enter__(self) -> "kernel_times":
        global _timed_calls
        from . import runtime
        if _timed_calls is not None:
            raise KernelError("kernel_times is already open")
        _timed_calls = []
        runtime.profile(True)
        return self

    def __exit__(self, *exc) -> None:
        global _timed_calls
        from . import runtime
        calls, _timed_calls = _timed_calls, None
        runtime.profile(False)                   # synchronises
        torch.cuda.synchronize()
        native = runtime.profile_results()
        self.calls = len(calls) + len(native)
        self.by_function = {}
        for name, start, end in calls:
            n, ms = self.by_function.get(name, (0, 0.0))
            self.by_function[name] = (n + 1, ms + start.elapsed_time(end))
        for name, ms_one, _ in native:
            n, ms = self.by_function.get(name, (0, 0.0))
            self.by_function[name] = (n + 1, ms + ms_one)
        self.total_ms = sum(ms for _, ms in self.by_function.values())
        self.idle_ms = sum(max(0.0, calls[i][2].elapsed_time(calls[i + 1][1])) for i in range(len(calls) - 1)) \
            + sum(idle for _, _, idle in native)

    def lines(self, what: str):
        """The report, most expensive first."""
        out = [f"profile {what}: {self.total_ms:.3f} ms of device time over {self.calls} kernel calls"]
        for name, (n, ms) in sorted(self.by_function.items(), key=lambda kv: -kv[1][1]):
            share = 100.0 * ms / self.total_ms if self.total_ms > 0 else 0.0
            out.append(f"profile:   {name} x{n} {ms:.3f} ms ({share:.1f}%)")
        out.append(f"profile {what}: idle {self.idle_ms:.3f} ms between timed calls")
        return out


def register_signature(lib: str, name: str, argtypes) -> None:
    _SIGNATURES[(lib, name)] = list(argtypes)


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r, :] = table[ids[r], :] widened to float32.  ids int32 [rows]; out float32 [rows, width]."""
    _cuda(table, ids, out)
    rows, width = out.shape
    _need(ids.dtype == torch.int32 and ids.numel() == rows, "embed: ids must be int32, one per output row")
    _need(out.dtype == torch.float32 and table.dim() == 2 and table.shape[1] == width, "embed: shapes do not fit")
    _check(_fn("rowwise", "llmx_embed")(_ptr(table), _code(table), _ptr(ids), _ptr(out), rows, width,
                                        table.shape[0], _stream()), "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            row_index: Optional[torch.Tensor] = None, zero: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = x[row_index[i] or i] * (rsqrt(mean x^2 + eps) * weight); x float32, out float32 or bfloat16.

    `zero` (optional): a float32 tensor the same launch clears (the output of a product that follows and
    adds its pieces with atomics)."""
    _cuda(x, weight, out, row_index, zero)
    if zero is not None:
        _need(zero.dtype == torch.float32 and zero.numel() % 4 == 0, "rmsnorm: the buffer to clear must be float32, a multiple of 4 long")
    rows, width = out.shape
    _need(x.dtype == torch.float32 and weight.dtype == torch.float32, "rmsnorm: input and weight must be float32")
    _need(x.dim() == 2 and x.shape[1] == width and weight.numel() == width, "rmsnorm: widths do not fit")
    if row_index is None:
        _need(x.shape[0] >= rows, "rmsnorm: fewer input rows than output rows")
    else:
        _need(row_index.dtype == torch.int32 and row_index.numel() == rows, "rmsnorm: row_index must be int32 per row")
    _check(_fn("rowwise", "llmx_rmsnorm")(_ptr(x), _ptr(weight), _ptr(out), _code(out), _ptr(row_index), rows, width,
                                          float(eps), _ptr(zero), 0 if zero is None else zero.numel(), _stream()),
           "rmsnorm")
    return out


def head_norm_rope_kv(qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                      q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                      cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                      slots: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor) -> None:
    """Per-head norm, rotation and the cache write for one layer.

    qkv float32 [rows, (heads + 2 kv_heads) * head_dim] (queries, keys, values);
    q_out [rows, heads * head_dim]; cache [pages, 2, kv_heads, page_size, head_dim];
    cos/sin float32 [positions, rot_half] or None (no rotation); slots int32 [rows],
    negative to skip a row's cache write.
    """
    _cuda(qkv, q_weight, k_weight, cos, sin, positions, slots, q_out, cache)
    rows = qkv.shape[0]
    q_w, kv_w = heads * head_dim, kv_heads * head_dim
    _need(qkv.dtype == torch.float32 and qkv.shape[1] == q_w + 2 * kv_w, "head_norm_rope_kv: qkv width does not fit")
    _need(tuple(q_out.shape) == (rows, q_w), "head_norm_rope_kv: q_out shape does not fit")
    _need(cache.dim() == 5 and cache.shape[1] == 2 and cache.shape[2] == kv_heads and cache.shape[4] == head_dim,
          "head_norm_rope_kv: cache layout does not fit")
    _need(positions.dtype == torch.int32 and slots.dtype == torch.int32 and positions.numel() >= rows
          and slots.numel() >= rows, "head_norm_rope_kv: positions and slots must be int32 per row")
    rot_half = 0
    if cos is not None:
        _need(sin is not None and cos.shape == sin.shape and cos.dtype == torch.float32 and cos.dim() == 2,
              "head_norm_rope_kv: cos and sin tables do not fit")
        rot_half = cos.shape[1]
        _need(2 * rot_half <= head_dim, "head_norm_rope_kv: rotated width exceeds the head width")
    for w in (q_weight, k_weight):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == head_dim), "head_norm_rope_kv: norm weight")
    page_size = cache.shape[3]
    _check(_fn("rowwise", "llmx_head_norm_rope_kv")(
        _ptr(qkv), qkv.shape[1], q_w, q_w + kv_w, _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin),
        rot_half, _ptr(positions), _ptr(slots), _ptr(q_out), _code(q_out), _ptr(cache), _code(cache), rows, heads,
        kv_heads, head_dim, page_size, _stream()), "head_norm_rope_kv")


def swiglu(gu: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = silu(gu[:, :F]) * gu[:, F:]; gu float32 [rows, 2F]."""
    _cuda(gu, out)
    rows, width = out.shape
    _need(gu.dtype == torch.float32 and tuple(gu.shape) == (rows, 2 * width), "swiglu: shapes do not fit")
    _check(_fn("rowwise", "llmx_swiglu")(_ptr(gu), _ptr(out), _code(out), rows, width, _stream()), "swiglu")
    return out


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out (+)= a @ w.T on the CUDA cores; a [M, K], w [N, K] of one type, out float32 [M, N]."""
    _cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    _need(w.shape[1] == k and tuple(out.shape) == (m, n) and out.dtype == torch.float32, "gemm: shapes do not fit")
    _need(a.dtype == w.dtype, "gemm: inputs and weights must have one element type")
    _check(_fn("gemm_plain", "llmx_gemm_plain")(_ptr(a), _code(a), _ptr(w), _code(w), _ptr(out), m, n, k,
                                                1 if accumulate else 0, _stream()), "gemm_plain")
    return out


def attention_plain(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, row_request: torch.Tensor,
                    positions: torch.Tensor, block_tables: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float) -> torch.Tensor:
    """Paged attention, one block per (row, head); q/out [rows, heads * head_dim] of one element type, the cache of
    its own (float32 or bfloat16 each)."""
    _cuda(q, cache, out, row_request, positions, block_tables)
    rows = q.shape[0]
    _need(q.shape == out.shape and q.shape[1] == heads * head_dim, "attention: q and out shapes do not fit")
    _need(q.dtype == out.dtype, "attention: q and out must have one element type")
    _need(cache.dim() == 5 and cache.shape[1] == 2 and cache.shape[2] == kv_heads and cache.shape[4] == head_dim,
          "attention: cache layout does not fit")
    for t in (row_request, positions, block_tables):
        _need(t.dtype == torch.int32, "attention: metadata must be int32")
    _need(block_tables.dim() == 2 and row_request.numel() >= rows and positions.numel() >= rows,
          "attention: metadata shapes do not fit")
    _check(_fn("attention_plain", "llmx_attention_plain")(
        _ptr(q), _code(q), _ptr(cache), _code(cache), _ptr(out), _ptr(row_request), _ptr(positions), _ptr(block_tables),
        block_tables.shape[1], rows, heads, kv_heads, head_dim, cache.shape[3], int(window or 0), float(scale),
        _stream()), "attention_plain")
    return out
