"""Python face of the paged attention kernels as the runtime dispatches them.

Requests of a step are split by how many rows they bring: those whose rows times the head ratio fit a 16-row
tile run the split-KV decode kernel (csrc/attention_decode.cu), the others a tiled prefill kernel (tcgen05,
csrc/attention_prefill_tc.cu, where the head width is 128; else warp-level,
csrc/attention_prefill.cu).  All read the same pages; which kernel a request runs depends only on its own row
count.  The dispatch and its launch plans are the native runtime's (`Attention::attend`, `llmx_plan_make` in
csrc/runtime/runtime.cpp); the functions here call them for tests and for callers that have queries already.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import runtime
from .ops import KernelError, _check, _cuda, _fn, _need, _ptr, register_signature

_i, _p, _ll = ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong
register_signature("attention_decode", "llmx_attn_cache_map", [_p, _p, _ll, _i, _i, _i])
register_signature("attention_decode", "llmx_attn_decode_cluster_merge", [_i])

PAGE = 16
WAVE_BLOCKS = 148 * 2            # decode blocks that run at once: two per SM
PREFILL_PART = 132               # floats of one (row, head, key range) partial result of the tcgen05 prefill kernel
PREFILL_MAX_PARTIAL = 1 << 26    # floats (256 MiB) the key ranges' partial results may take


def supported(heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tiled bfloat16 kernels take this shape (else the plain kernel runs)."""
    return runtime.tiled_attention(heads, kv_heads, head_dim, page_size) > 0


def tensor_core_prefill(heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether prompt portions run the tcgen05 kernel (head width 128, up to 16 query heads a kv head)."""
    return runtime.tiled_attention(heads, kv_heads, head_dim, page_size) == 2


def decode_schedule(n_requests: int, kv_heads: int, max_context: int, head_dim: int = 128) -> Tuple[int, int]:
    """(key ranges, keys per range) for requests that bring few rows (the runtime's `decode_schedule`)."""
    return runtime.decode_schedule(n_requests, kv_heads, max_context, head_dim)


def prefill_shape(n_requests: int, kv_heads: int, ratio: int, max_rows: int, max_context: int, window: int,
                  sms: int = 148) -> Tuple[int, int]:
    """(row tiles an item, key ranges) for the tcgen05 prefill kernel (the runtime's `prefill_shape`)."""
    return runtime.prefill_shape(n_requests, kv_heads, ratio, max_rows, max_context, window, sms)


def cluster_merge(on: bool) -> bool:
    """Up to sixteen key ranges of a (request, kv head) are launched as one thread-block cluster and combined through
    its shared memory (on, the default); off, they are combined like more ranges, through memory and a counter.
    Returns the setting before."""
    runtime.need("attention_decode")
    before = bool(_fn("attention_decode", "llmx_attn_decode_cluster_merge")(1 if on else 0))
    runtime.lib().llmx_rt_reset_caches()          # the runtime asks the kernels again which clusters fit
    return before


class CacheMap:
    """The TMA descriptor of one cache entry's storage [pages, 2, kv_heads, 16, head_dim], for callers that launch
    the decode kernel themselves."""

    def __init__(self, cache: torch.Tensor):
        self.cache = cache
        self._raw = ctypes.create_string_buffer(128 + 64)
        self.address = (ctypes.addressof(self._raw) + 63) & ~63
        pages, _, kv_heads, page_size, head_dim = cache.shape
        _check(_fn("attention_decode", "llmx_attn_cache_map")(ctypes.c_void_p(self.address), _ptr(cache), pages,
                                                              kv_heads, page_size, head_dim), "attention cache map", 0)


def cache_map(cache: torch.Tensor) -> CacheMap:
    return CacheMap(cache)


class OneEntryCache:
    """A cache of one key/value entry, as the runtime wants to see it (for tests that bring their own storage)."""

    def __init__(self, storage: torch.Tensor):
        self.storage = storage
        self.views = runtime.CacheViews(1)
        self.views.set_kv(0, 0, storage)

    def entry_storage(self, entry: int):
        return 0, self.storage


def _struct(step, entry_cache: Optional[OneEntryCache], workspace: int = 0):
    s = step.struct_for(None, workspace)
    if entry_cache is not None:
        s.caches = entry_cache.views.handle
    return s


def paged_attention(q: torch.Tensor, out: torch.Tensor, step, cache_entry: int, heads: int, kv_heads: int,
                    head_dim: int, window: Optional[int], scale: float, cache: Optional[OneEntryCache] = None) -> None:
    """out = attention of the step's rows over a cache entry; q/out [rows, heads * head_dim].  `step` must carry a
    launch plan for this shape when the tiled kernels take it (engine.batch.single_group_step makes one)."""
    _cuda(q, out)
    _need(q.shape == out.shape and q.shape[1] == heads * head_dim and q.dtype == out.dtype, "attention: q and out shapes do not fit")
    rt = runtime.lib()
    probe = _struct(step, cache)
    need = rt.llmx_paged_attention_workspace(ctypes.byref(probe), cache_entry, heads, kv_heads, head_dim, int(window or 0))
    runtime.bind_missing()
    s = _struct(step, cache, need)
    runtime.check(rt.llmx_paged_attention(ctypes.byref(s), q.data_ptr(), runtime.code(q.dtype), cache_entry, out.data_ptr(),
                                          heads, kv_heads, head_dim, int(window or 0), float(scale)), "attention")


def decode_from_qkv(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                    cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], out: torch.Tensor, step, cache_entry: int,
                    heads: int, kv_heads: int, head_dim: int, window: Optional[int], scale: float,
                    cache: Optional[OneEntryCache] = None) -> bool:
    """Attention for a step in which every request brings few rows, straight from the q/k/v product's float32
    output: the decode kernel's blocks norm and rotate their own queries, and the new keys and values are
    stored (and used) by the blocks whose key range holds them.  Returns False, having done nothing, when the
    step or the shapes do not qualify."""
    _cuda(qkv, q_weight, k_weight, cos, sin, out)
    _need(qkv.dtype is torch.float32 and qkv.shape[1] == (heads + 2 * kv_heads) * head_dim
          and tuple(out.shape) == (qkv.shape[0], heads * head_dim) and out.dtype is torch.bfloat16,
          "attention: the product's output and the attention output do not fit the head counts")
    rt = runtime.lib()
    probe = _struct(step, cache)
    need = rt.llmx_paged_attention_workspace(ctypes.byref(probe), cache_entry, heads, kv_heads, head_dim, int(window or 0))
    runtime.bind_missing()
    s = _struct(step, cache, need)
    status = rt.llmx_decode_from_qkv(ctypes.byref(s), qkv.data_ptr(), cache_entry, runtime.ptr(q_weight), runtime.ptr(k_weight),
                                     float(eps), runtime.ptr(cos), runtime.ptr(sin), 0 if cos is None else cos.shape[1],
                                     out.data_ptr(), heads, kv_heads, head_dim, int(window or 0), float(scale))
    if status == -1:
        return False
    runtime.check(status, "attention")
    return True


def attention_step(device, layout_rows, tables, heads: int, kv_heads: int, head_dim: int, window: Optional[int],
                   page_size: int = PAGE):
    """A step of (history, rows) pairs over ready block tables [requests, max_pages] with the launch plan of an
    attention of this shape: what `paged_attention` and `decode_from_qkv` want (tests, callers with queries of their own).
    `step.plan.native.plan` offers `force_decode` and `force_prefill_shape`."""
    from .engine.batch import single_group_step
    from .parts.base import NativeHandle
    shape = NativeHandle(runtime.lib().llmx_attention_shape(heads, kv_heads, head_dim, int(window or 0)))
    if supported(heads, kv_heads, head_dim, page_size):
        runtime.need("attention_decode")      # its launch plans ask the device which clusters fit
    return single_group_step(device, layout_rows, tables, page_size, plan_parts=[shape.handle])


def paged_attention_bf16(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, step, group, heads: int,
                         kv_heads: int, head_dim: int, window: Optional[int], scale: float) -> None:
    """`paged_attention` over a storage tensor [pages, 2, kv_heads, page_size, head_dim] the caller brings."""
    paged_attention(q, out, step, 0, heads, kv_heads, head_dim, window, scale, cache=OneEntryCache(cache))
