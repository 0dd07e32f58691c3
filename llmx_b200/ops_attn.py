"""Python face of the tiled bfloat16 attention kernels (csrc/attention_decode.cu, csrc/attention_prefill.cu).

Requests of a step are split by how many rows they bring: those whose rows times the head ratio
fit a 16-row tile run the split-KV decode kernel, the others the tiled prefill kernel.  Both
read the same pages; which kernel a request runs depends only on its own row count.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from .ops import KernelError, _check, _cuda, _fn, _need, _ptr, _stream, register_signature
from .ops_tc import error_word

_i, _p, _f, _ll = ctypes.c_int, ctypes.c_void_p, ctypes.c_float, ctypes.c_longlong
register_signature("attention_decode", "llmx_attn_cache_map", [_p, _p, _ll, _i, _i, _i])
register_signature("attention_decode", "llmx_attn_decode",
                   [_p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _p, _i, _i, _p, _p])
register_signature("attention_decode", "llmx_attn_decode_fused",
                   [_p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _p, _i, _i, _p, _p, _p])
# cache_map, qkv, stride, k_offset, v_offset, q_weight, k_weight, eps, cos, sin, slots, cache, out, partial, req_list,
# n_req, row_start, row_count, history, tables, table_stride, heads, kv_heads, head_dim, page, window, scale, splits,
# chunk_ptr, chunk, max_rows, counters, error_word, stream
register_signature("attention_decode", "llmx_attn_decode_qkv",
                   [_p, _p, _i, _i, _i, _p, _p, _f, _p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i,
                    _i, _f, _i, _p, _i, _i, _p, _p, _p])
register_signature("attention_decode", "llmx_attn_decode_cluster_merge", [_i])
register_signature("attention_decode", "llmx_attn_decode_max_clusters", [_i, _i])
register_signature("attention_prefill_tc", "llmx_attn_prefill_tc_cache_map", [_p, _p, _ll, _i, _i, _i])
register_signature("attention_prefill_tc", "llmx_attn_prefill_tc",
                   [_p, _p, _p, _i, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _p, _p, _p])
register_signature("attention_prefill", "llmx_attn_prefill",
                   [_p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _p, _p])

PAGE = 16
WAVE_BLOCKS = 148 * 2            # decode blocks that run at once: two per SM


def supported(heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    return head_dim in (64, 128) and page_size == PAGE and heads % kv_heads == 0 and heads // kv_heads <= 16


class CacheMap:
    """The TMA descriptor of one cache entry's storage [pages, 2, kv_heads, 16, head_dim]."""

    def __init__(self, cache: torch.Tensor):
        self.cache = cache
        self._raw = ctypes.create_string_buffer(128 + 64)
        self.address = (ctypes.addressof(self._raw) + 63) & ~63
        pages, _, kv_heads, page_size, head_dim = cache.shape
        _check(_fn("attention_decode", "llmx_attn_cache_map")(ctypes.c_void_p(self.address), _ptr(cache), pages,
                                                              kv_heads, page_size, head_dim), "attention cache map", 0)


class CacheHalfMap:
    """The descriptor the tcgen05 prefill kernel reads the same storage through (boxes of half a page-head)."""

    def __init__(self, cache: torch.Tensor):
        self.cache = cache
        self._raw = ctypes.create_string_buffer(128 + 64)
        self.address = (ctypes.addressof(self._raw) + 63) & ~63
        pages, _, kv_heads, page_size, head_dim = cache.shape
        _check(_fn("attention_prefill_tc", "llmx_attn_prefill_tc_cache_map")(
            ctypes.c_void_p(self.address), _ptr(cache), pages, kv_heads, page_size, head_dim), "attention cache map", 0)


_half_maps: Dict[int, CacheHalfMap] = {}


def cache_half_map(cache: torch.Tensor) -> CacheHalfMap:
    m = _half_maps.get(cache.data_ptr())
    if m is None or m.cache.shape != cache.shape:
        m = CacheHalfMap(cache)
        _half_maps[cache.data_ptr()] = m
    return m


def tensor_core_prefill(heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether prompt portions run the tcgen05 kernel (head width 128, a head ratio dividing 128)."""
    return head_dim == 128 and page_size == PAGE and heads % kv_heads == 0 and 128 % (heads // kv_heads) == 0


_maps: Dict[int, CacheMap] = {}
_counters: Dict[int, torch.Tensor] = {}
MAX_COUNTERS = 65536


def _counter_buffer(device) -> torch.Tensor:
    """Ints (one per request and kv head) the decode kernel's blocks count themselves into; every launch
    leaves them zero."""
    idx = torch.device(device).index or 0
    c = _counters.get(idx)
    if c is None:
        c = torch.zeros(MAX_COUNTERS, dtype=torch.int32, device=device)
        _counters[idx] = c
    return c


def cache_map(cache: torch.Tensor) -> CacheMap:
    m = _maps.get(cache.data_ptr())
    if m is None or m.cache.shape != cache.shape:
        m = CacheMap(cache)
        _maps[cache.data_ptr()] = m
    return m


def cluster_merge(on: bool) -> bool:
    """Up to sixteen key ranges of a (request, kv head) are launched as one thread-block cluster and combined through
    its shared memory (on, the default); off, they are combined like more ranges, through memory and a counter.
    Returns the setting before."""
    _cluster_counts.clear()
    return bool(_fn("attention_decode", "llmx_attn_decode_cluster_merge")(1 if on else 0))


# Clusters of 2..16 decode blocks (head width 128) that a B200 runs at once: what is assumed where the device
# cannot be asked (no GPU at hand); `max_clusters` asks it.
_B200_CLUSTERS = {2: 148, 3: 93, 4: 71, 5: 56, 6: 45, 7: 37, 8: 33, 12: 21, 16: 14}
_cluster_counts: Dict[Tuple[int, int], int] = {}
CLUSTER_FILL = 0.92            # of the clusters that fit at once, as many are planned for


def max_clusters(head_dim: int, size: int) -> int:
    """Clusters of `size` decode blocks the device runs at once (0: clusters are turned off or cannot run)."""
    key = (head_dim, size)
    if key not in _cluster_counts:
        try:
            n = int(_fn("attention_decode", "llmx_attn_decode_max_clusters")(head_dim, size))
        except Exception:               # no compiler
            n = -1
        if n < 0:                       # no device to ask: plan as for a B200
            return _B200_CLUSTERS.get(size, 0) * (2 if head_dim == 64 else 1)
        _cluster_counts[key] = n
    return _cluster_counts[key]


def decode_schedule(n_requests: int, kv_heads: int, max_context: int, head_dim: int = 128) -> Tuple[int, int]:
    """(key ranges, keys per range) for requests that bring few rows.

    Up to sixteen ranges of a (request, kv head) run as one thread-block cluster and meet in its shared memory; more
    would meet through memory and a counter, which costs about 4 us more a launch.  A cluster starts only when
    all its blocks find room in one part of the chip, so no more clusters are planned than the device runs at once
    (with a margin: 32 clusters of 8 where 33 fit ran slower than 32 of 6): a second round would double the kernel's
    time.  Measured on a B200 inside the decode step (32 heads over 8; 1 to 16 requests, 1,024 to 32,768 keys) and
    alone (512 to 32,768 keys): one range per 128 keys below 1,024 keys; then as many as fit, eight at most below
    4,096 keys, sixteen from there on (one request: 3.54 -> 3.37 ms a step at 8,192 keys), twelve where sixteen do
    not fit only from 16,384 keys on."""
    blocks = max(n_requests * kv_heads, 1)
    wave = WAVE_BLOCKS // blocks
    if max_context < 1024:
        want, sizes = max(1, max_context // 128), (8, 6, 4, 3, 2)
    elif max_context < 4096:
        want, sizes = 8, (8, 6, 4, 3, 2)
    elif max_context < 16384:
        want, sizes = 16, (16, 8, 6, 4, 3, 2)
    else:
        want, sizes = 16, (16, 12, 8, 6, 4, 3, 2)
    if max_clusters(head_dim, 2) > 0:
        splits = next((s for s in sizes if s <= want and blocks <= CLUSTER_FILL * max_clusters(head_dim, s)), 1)
    else:                          # clusters turned off: ranges meet through memory, a wave of blocks at most
        splits = max(1, min(wave, want if max_context >= 16384 else min(want, 8)))
    chunk = -(-(-(-max_context // 64)) // splits) * 64
    splits = max(1, -(-max_context // chunk))
    return splits, chunk


PREFILL_PART = 132             # floats of one (row, head, key range) partial result of the tcgen05 prefill kernel
PREFILL_MAX_PARTIAL = 1 << 26  # floats (256 MiB) the key ranges' partial results may take


def prefill_shape(n_requests: int, kv_heads: int, ratio: int, max_rows: int, max_context: int, window: int,
                  sms: int = 148) -> Tuple[int, int]:
    """(row tiles an item, key ranges) for the tcgen05 prefill kernel.  Its work items are (request, kv head, block of
    rows); a block of threads walks an item's key stages one after the other, so when items are fewer than the SMs
    the longest item is the kernel's time.  Two row tiles an item share their key stages and keep the tensor core
    busier (about 1.05 us a tile and stage of 128 keys against 1.9 us for a tile alone); cutting the keys into
    ranges makes more, shorter items at the price of a second small kernel that adds the ranges up.  The estimate
    below takes the cheapest of the combinations."""
    per_tile = max(1, 128 // ratio)
    reach = min(max_context, window + max_rows) if window else max_context
    stages = -(-reach // 128)
    best = None
    for tiles, rate in ((2, 2.1), (1, 1.9)):
        items = -(-max_rows // (tiles * per_tile)) * kv_heads * n_requests
        for splits in (1, 2, 3, 4, 6, 8):
            if splits > 1 and (stages < 8 * splits or max_rows * kv_heads * ratio * n_requests * splits * PREFILL_PART
                               > PREFILL_MAX_PARTIAL):
                break
            t = -(-items * splits // sms) * -(-stages // splits) * rate + (6.0 if splits > 1 else 0.0)
            if best is None or t < best[0] - 1e-9:
                best = (t, tiles, splits)
    return best[1], best[2]


def _request_lists(step, max_rows: int):
    """Device lists of the requests that bring at most `max_rows` rows and of the others (cached on the step)."""
    key = ("attn_lists", max_rows)
    got = step.extras.get(key)
    if got is None:
        small = [r for r, n in enumerate(step.host_row_count) if n <= max_rows]
        large = [r for r, n in enumerate(step.host_row_count) if n > max_rows]
        host = torch.tensor(small + large + [0], dtype=torch.int32).pin_memory()
        dev = host.to(step.token_ids.device, non_blocking=True)
        ctx_small = max((step.host_history[r] + step.host_row_count[r] for r in small), default=0)
        rows_large = max((step.host_row_count[r] for r in large), default=0)
        rows_small = max((step.host_row_count[r] for r in small), default=0)
        got = (dev[:len(small)], len(small), ctx_small, rows_small, dev[len(small):len(small) + len(large)],
               len(large), rows_large)
        step.extras[key] = got
    return got


def decoding_rows_only(step, heads: int, kv_heads: int) -> bool:
    """Whether every request of the step brings so few rows that the decode kernel serves them all."""
    lists = _request_lists(step, 16 // (heads // kv_heads))
    return lists[1] > 0 and lists[5] == 0


def paged_attention_bf16(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, step, group, heads: int,
                         kv_heads: int, head_dim: int, window: Optional[int], scale: float) -> None:
    _cuda(q, cache, out)
    _need(q.dtype is torch.bfloat16 and cache.dtype is torch.bfloat16 and out.dtype is torch.bfloat16,
          "attention: bfloat16 queries, cache and output")
    _need(q.shape == out.shape and q.shape[1] == heads * head_dim, "attention: q and out shapes do not fit")
    ratio = heads // kv_heads
    max_rows = 16 // ratio
    cmap = cache_map(cache)
    tables = group.block_tables
    (small, n_small, ctx_small, rows_small, large, n_large, rows_large) = _request_lists(step, max_rows)
    err = error_word(q.device)
    win = int(window or 0)
    if n_small:
        sched = step.extras.get("decode_schedule")
        if sched is None:
            splits, chunk = decode_schedule(n_small, kv_heads, ctx_small, head_dim)
            chunk_ptr = None
        else:                      # a recorded step: the grid is fixed, the keys per range come from the device
            splits, chunk, chunk_ptr = sched
        partial = None
        if splits > 1:
            key = ("attn_partial", splits, heads, head_dim)
            partial = step.extras.get(key)
            if partial is None:
                partial = torch.empty((q.shape[0] * heads * splits * (head_dim + 2),), dtype=torch.float32,
                                      device=q.device)
                step.extras[key] = partial
        counters = _counter_buffer(q.device) if splits > 1 and n_small * kv_heads <= MAX_COUNTERS else None
        _check(_fn("attention_decode", "llmx_attn_decode_fused")(
            ctypes.c_void_p(cmap.address), _ptr(q), _ptr(out), _ptr(partial), _ptr(small), n_small,
            _ptr(step.row_start), _ptr(step.row_count), _ptr(step.history), _ptr(tables), tables.shape[1], heads,
            kv_heads, head_dim, cache.shape[3], win, float(scale), splits, _ptr(chunk_ptr), chunk, max(rows_small, 1),
            _ptr(counters), _ptr(err), _stream()), "attention_decode", 2 if splits > 1 and counters is None else 1)
    if n_large and tensor_core_prefill(heads, kv_heads, head_dim, cache.shape[3]) and not step.extras.get("no_tc_attention"):
        hmap = cache_half_map(cache)
        shape = step.extras.get("attn_prefill_shape")          # forced by a test, else chosen once a step and mixer shape
        if shape is None:
            key = ("attn_prefill_shape", kv_heads, ratio, win)
            shape = step.extras.get(key)
            if shape is None:
                ctx_large = max(step.host_history[r] + n for r, n in enumerate(step.host_row_count) if n > max_rows)
                shape = step.extras[key] = prefill_shape(n_large, kv_heads, ratio, rows_large, ctx_large, win)
        tiles, splits = shape
        partial = None
        if splits > 1:
            key = ("attn_prefill_partial", splits, heads)
            partial = step.extras.get(key)
            if partial is None:
                partial = torch.empty((q.shape[0] * heads * splits * PREFILL_PART,), dtype=torch.float32, device=q.device)
                step.extras[key] = partial
        _check(_fn("attention_prefill_tc", "llmx_attn_prefill_tc")(
            ctypes.c_void_p(hmap.address), _ptr(q), _ptr(out), q.shape[0], _ptr(large), n_large, _ptr(step.row_start),
            _ptr(step.row_count), _ptr(step.history), _ptr(tables), tables.shape[1], heads, kv_heads, head_dim,
            cache.shape[3], win, float(scale), rows_large, tiles, splits, _ptr(partial), _ptr(err), _stream()),
            "attention_prefill_tc", 2 if splits > 1 else 1)
    elif n_large:
        _check(_fn("attention_prefill", "llmx_attn_prefill")(
            ctypes.c_void_p(cmap.address), _ptr(q), _ptr(out), _ptr(large), n_large, _ptr(step.row_start),
            _ptr(step.row_count), _ptr(step.history), _ptr(tables), tables.shape[1], heads, kv_heads, head_dim,
            cache.shape[3], win, float(scale), rows_large, _ptr(err), _stream()), "attention_prefill")


def decode_from_qkv(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                    cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], slots: torch.Tensor,
                    cache: torch.Tensor, out: torch.Tensor, step, group, heads: int, kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float) -> bool:
    """Attention for a step in which every request brings few rows, straight from the q/k/v product's float32
    output: the decode kernel's blocks norm and rotate their own queries, and the new keys and values are
    stored (and used) by the blocks whose key range holds them, so the separate norm / rotation / cache-write
    kernel does not run.  Returns False, having done nothing, when the step or the shapes do not qualify."""
    if (head_dim != 128 or cache.shape[3] != PAGE or cache.dtype is not torch.bfloat16 or out.dtype is not torch.bfloat16
            or qkv.dtype is not torch.float32 or not supported(heads, kv_heads, head_dim, cache.shape[3])
            or step.extras.get("no_qkv_attention")):
        return False
    if cos is not None and (cos.shape[1] != 64 or sin is None):
        return False
    ratio = heads // kv_heads
    (small, n_small, ctx_small, rows_small, large, n_large, rows_large) = _request_lists(step, 16 // ratio)
    if n_large or not n_small or n_small * kv_heads > MAX_COUNTERS:
        return False
    _cuda(qkv, q_weight, k_weight, cos, sin, slots, cache, out)
    _need(qkv.shape[1] == (heads + 2 * kv_heads) * head_dim and out.shape == (qkv.shape[0], heads * head_dim),
          "attention: the product's output and the attention output do not fit the head counts")
    sched = step.extras.get("decode_schedule")
    if sched is None:
        splits, chunk = decode_schedule(n_small, kv_heads, ctx_small, head_dim)
        chunk_ptr = None
    else:
        splits, chunk, chunk_ptr = sched
    partial = None
    if splits > 1:
        key = ("attn_partial", splits, heads, head_dim)
        partial = step.extras.get(key)
        if partial is None:
            partial = torch.empty((qkv.shape[0] * heads * splits * (head_dim + 2),), dtype=torch.float32, device=qkv.device)
            step.extras[key] = partial
    cmap = cache_map(cache)
    tables = group.block_tables
    _check(_fn("attention_decode", "llmx_attn_decode_qkv")(
        ctypes.c_void_p(cmap.address), _ptr(qkv), qkv.shape[1], heads * head_dim, (heads + kv_heads) * head_dim,
        _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), _ptr(slots), _ptr(cache), _ptr(out),
        _ptr(partial), _ptr(small), n_small, _ptr(step.row_start), _ptr(step.row_count), _ptr(step.history),
        _ptr(tables), tables.shape[1], heads, kv_heads, head_dim, cache.shape[3], int(window or 0), float(scale), splits,
        _ptr(chunk_ptr), chunk, max(rows_small, 1), _ptr(_counter_buffer(qkv.device)), _ptr(error_word(qkv.device)),
        _stream()), "attention_decode")
    return True
