"""Python face of the native runtime (csrc/runtime/): the parts' forward passes, launch plans, the model's forward.

The runtime is host code in C++ (csrc/runtime/llmx_runtime.h).  This module loads it, hands it the kernel
libraries' entry points as they are needed, and wraps its objects:

    Step        the `llmx_step` description of one step (made from a `StepBatch`)
    Plan        launch decisions of a step's shape (`llmx_plan_*`)
    need(lib)   build and load a kernel library and bind its functions into the runtime

Kernel libraries are bound lazily: the runtime's dry run of a forward pass (which also sizes the step's
workspace) reports the entry points it would call and does not have; their libraries are then built, loaded
and bound, so a run compiles only what its model, precision and shapes use.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .csrc import build as _build

F32, BF16 = 0, 1
MAX_GROUPS = 8
COUNTERS = 65536
FLAG_INVARIANT = 1

_i, _f, _p, _ll, _sz = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_size_t


class KernelError(RuntimeError):
    """A kernel or the runtime refused its arguments, or a launch failed."""


class StepStruct(ctypes.Structure):
    _fields_ = [("rows", _i), ("requests", _i), ("wanted", _i), ("groups", _i), ("position_streams", _i), ("room", _i),
                ("meta", _p),
                ("token_ids", _i), ("positions", _i), ("row_request", _i), ("row_start", _i), ("row_count", _i),
                ("history", _i), ("state_slots", _i), ("logit_rows", _i), ("state_slots_out", _i),
                ("block_tables", _i * MAX_GROUPS), ("table_stride", _i * MAX_GROUPS), ("slots", _i * MAX_GROUPS),
                ("page_size", _i * MAX_GROUPS),
                ("plan_offset", _i), ("plan", _p), ("caches", _p), ("workspace", _p), ("workspace_bytes", _sz),
                ("error_word", _p), ("counters", _p), ("stream", _p)]


class LinearDesc(ctypes.Structure):
    _fields_ = [("weight", _p), ("dtype", _i), ("out_features", _i), ("in_features", _i), ("flags", _i)]


class AttentionDesc(ctypes.Structure):
    _fields_ = [("hidden", _i), ("heads", _i), ("kv_heads", _i), ("head_dim", _i), ("window", _i),
                ("scale", _f), ("qk_norm_eps", _f), ("q_norm", _p), ("k_norm", _p), ("cos", _p), ("sin", _p),
                ("rot_half", _i), ("table_positions", _i), ("position_stream", _i),
                ("qkv", LinearDesc), ("o", LinearDesc), ("flags", _i)]


class MlpDesc(ctypes.Structure):
    _fields_ = [("hidden", _i), ("intermediate", _i), ("gate_up", LinearDesc), ("down", LinearDesc), ("flags", _i)]


class LayerStepStruct(ctypes.Structure):
    _fields_ = [("block", _i), ("cache_entry", _i), ("write_cache", _i)]


_SP = ctypes.POINTER(StepStruct)
_SIGNATURES = {
    "llmx_rt_version": (_i, []),
    "llmx_rt_bind": (_i, [ctypes.c_char_p, _p]),
    "llmx_rt_load_kernels": (_i, [ctypes.c_char_p]),
    "llmx_rt_last_error": (ctypes.c_char_p, []),
    "llmx_rt_launches": (_ll, []),
    "llmx_rt_count_launches": (None, [_ll]),
    "llmx_rt_profile": (_i, [_i]),
    "llmx_rt_profile_read": (_i, [_i, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(_f), ctypes.POINTER(_f)]),
    "llmx_rt_fail_call": (None, [ctypes.c_char_p, _i]),
    "llmx_rt_missing": (_i, [_i, ctypes.POINTER(ctypes.c_char_p)]),
    "llmx_rt_reset_caches": (None, []),
    "llmx_rt_pair_products": (_i, [_i]),
    "llmx_gemm_plan": (None, [_i, _i, _i, _i, _i, ctypes.POINTER(_i), ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "llmx_heads_tile": (_i, [_i, _i, _i, _i]),
    "llmx_decode_schedule": (None, [_i, _i, _i, _i, _p, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "llmx_prefill_shape": (None, [_i, _i, _i, _i, _i, _i, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "llmx_tiled_attention": (_i, [_i, _i, _i, _i]),
    "llmx_caches_create": (_p, [_i]),
    "llmx_caches_destroy": (None, [_p]),
    "llmx_caches_set_kv": (_i, [_p, _i, _i, _p, _i, _ll, _i, _i, _i]),
    "llmx_caches_set_state": (_i, [_p, _i, _p, _ll, _ll]),
    "llmx_plan_make": (_p, [_p, _p, _i, _p, _p, _i, _i, _i]),
    "llmx_plan_ints": (_i, [_p]),
    "llmx_plan_fill": (_i, [_p, _p, _p]),
    "llmx_plan_free": (None, [_p]),
    "llmx_plan_force_prefill_shape": (None, [_p, _i, _i]),
    "llmx_plan_force_decode": (None, [_p, _i, _i]),
    "llmx_plan_describe": (_i, [_p, _p]),
    "llmx_rmsnorm_create": (_p, [_p, _i, _f, _i]),
    "llmx_attention_create": (_p, [ctypes.POINTER(AttentionDesc)]),
    "llmx_gated_mlp_create": (_p, [ctypes.POINTER(MlpDesc)]),
    "llmx_linear_create": (_p, [ctypes.POINTER(LinearDesc)]),
    "llmx_prenorm_block_create": (_p, [_p, _p, _p, _p]),
    "llmx_callback_create": (_p, [_i, _p, _p, _i]),
    "llmx_embedding_create": (_p, [_p, _i, _i, _i]),
    "llmx_head_create": (_p, [_p, ctypes.POINTER(LinearDesc)]),
    "llmx_part_destroy": (None, [_p]),
    "llmx_attention_set_tables": (_i, [_p, _p, _p, _i, _i]),
    "llmx_norm_forward": (_i, [_p, _SP, _p, _p, _i, _p, _i, _p, _ll]),
    "llmx_mixer_forward": (_i, [_p, _SP, _p, _i, _i, _p, _i, _p]),
    "llmx_ffn_forward": (_i, [_p, _SP, _p, _i, _p, _p]),
    "llmx_block_forward": (_i, [_p, _SP, _p, _i, _i, _i]),
    "llmx_embedding_forward": (_i, [_p, _SP, _p, _p, _i]),
    "llmx_head_forward": (_i, [_p, _SP, _p, _p]),
    "llmx_linear_forward": (_i, [_p, _SP, _p, _i, _p, _i, _i]),
    "llmx_linear_gated": (_i, [_p, _SP, _p, _i, _p]),
    "llmx_part_wants_cleared": (_ll, [_p, _SP, _i]),
    "llmx_linear_adds_pieces": (_i, [_p, _i]),
    "llmx_part_workspace": (_sz, [_p, _SP, _i, _i]),
    "llmx_attention_shape": (_p, [_i, _i, _i, _i]),
    "llmx_paged_attention": (_i, [_SP, _p, _i, _i, _p, _i, _i, _i, _i, _f]),
    "llmx_paged_attention_workspace": (_sz, [_SP, _i, _i, _i, _i, _i]),
    "llmx_decode_from_qkv": (_i, [_SP, _p, _i, _p, _p, _f, _p, _p, _i, _p, _i, _i, _i, _i, _f]),
    "llmx_model_create": (_p, [_p, _p, _i, _p, _i, _p, _i, _i]),
    "llmx_model_destroy": (None, [_p]),
    "llmx_model_workspace": (_sz, [_p, _SP]),
    "llmx_model_forward": (_i, [_p, _SP, _p]),
}

# Which library exports which entry point the runtime calls.
KERNEL_LIBS: Dict[str, str] = {
    "llmx_embed": "rowwise", "llmx_rmsnorm": "rowwise", "llmx_head_norm_rope_kv": "rowwise", "llmx_swiglu": "rowwise",
    "llmx_gemm_plain": "gemm_plain", "llmx_attention_plain": "attention_plain",
    "llmx_gemm_tc_weight_map": "gemm_tc", "llmx_gemm_tc_weight_map_box": "gemm_tc", "llmx_gemm_tc": "gemm_tc",
    "llmx_gemm_tc_swiglu": "gemm_tc", "llmx_gemm_tc_heads": "gemm_tc", "llmx_gemm_tc_pair": "gemm_tc_pair",
    "llmx_gemm_tc_pair_swiglu": "gemm_tc_pair", "llmx_gemm_tc_pair_heads": "gemm_tc_pair",
    "llmx_attn_cache_map": "attention_decode", "llmx_attn_decode_fused": "attention_decode",
    "llmx_attn_decode_qkv": "attention_decode", "llmx_attn_decode_max_clusters": "attention_decode",
    "llmx_attn_prefill_tc_cache_map": "attention_prefill_tc", "llmx_attn_prefill_tc": "attention_prefill_tc",
    "llmx_attn_prefill": "attention_prefill",
    "llmx_sample": "sampling", "llmx_penalize": "sampling",
}

_lib = None
_bound_libs = set()


def lib():
    """The loaded runtime library (built on first use)."""
    global _lib
    if _lib is None:
        rt = _build.load("runtime")
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(rt, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = rt
    return _lib


def last_error() -> str:
    return (lib().llmx_rt_last_error() or b"").decode("utf-8", "replace")


def check(status: int, what: str = "") -> None:
    if status:
        raise KernelError(f"{what + ': ' if what else ''}{last_error() or 'error ' + str(status)}")


def need(library: str) -> None:
    """Build and load a kernel library and bind the entry points the runtime calls from it."""
    if library in _bound_libs:
        return
    loaded = _build.load(library)
    rt = lib()
    for name, owner in KERNEL_LIBS.items():
        if owner == library:
            check(rt.llmx_rt_bind(name.encode(), ctypes.cast(getattr(loaded, name), _p)), "binding " + name)
    _bound_libs.add(library)
    rt.llmx_rt_reset_caches()


def bind_missing() -> bool:
    """Bind the entry points the runtime's last dry run found unbound; True if there were any."""
    rt = lib()
    names, k = [], 0
    name = ctypes.c_char_p()
    while rt.llmx_rt_missing(k, ctypes.byref(name)):
        names.append(name.value.decode())
        k += 1
    for n in names:
        need(KERNEL_LIBS[n])
    if names:
        rt.llmx_rt_reset_caches()
    return bool(names)


def fail_call(name: Optional[str], nth: int = 1) -> None:
    """The nth call from now of kernel entry point `name` fails on the host, before anything is launched (for tests
    of what a failed step leaves behind); `None` withdraws a pending failure."""
    lib().llmx_rt_fail_call(name.encode() if name else None, int(nth))


def launches() -> int:
    return int(lib().llmx_rt_launches()) if _lib is not None else 0


def count_launches(n: int) -> None:
    lib().llmx_rt_count_launches(int(n))


def code(dtype: torch.dtype) -> int:
    if dtype is torch.float32:
        return F32
    if dtype is torch.bfloat16:
        return BF16
    raise KernelError(f"element type {dtype} is not one the kernels take (float32, bfloat16)")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def current_stream() -> int:
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


# ---- per-device buffers the kernels share -------------------------------------------------------------------
_error_words: Dict[int, torch.Tensor] = {}
_counters: Dict[int, torch.Tensor] = {}
_ERROR_NAMES = {101: "the TMA producer waited for a free stage", 102: "the MMA issuer waited for a loaded stage",
                103: "the MMA issuer waited for a free accumulator", 104: "the epilogue waited for an accumulator",
                105: "a test kernel's consumer waited for a barrier nobody arrives at"}


def error_word(device) -> torch.Tensor:
    """The device int a kernel records a failed (bounded) wait in, one per device."""
    idx = torch.device(device).index or 0
    w = _error_words.get(idx)
    if w is None:
        w = _error_words[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return w


def counters(device) -> torch.Tensor:
    """Ints (one per request and kv head) the decode kernel's blocks count themselves into; every launch leaves them zero."""
    idx = torch.device(device).index or 0
    c = _counters.get(idx)
    if c is None:
        c = _counters[idx] = torch.zeros(COUNTERS, dtype=torch.int32, device=device)
    return c


def check_errors() -> None:
    """Raise if any kernel gave up a wait (synchronises the devices that ran one)."""
    for idx, w in _error_words.items():
        c = int(w.item())
        if c:
            w.zero_()
            raise KernelError(f"a kernel on device {idx} gave up a bounded wait: {_ERROR_NAMES.get(c, c)}")


# ---- launch decisions (one implementation, in the runtime) --------------------------------------------------
def gemm_plan(m: int, n: int, k: int, accumulate: bool, sms: int = 0):
    s, t, r = _i(), _i(), _i()
    lib().llmx_gemm_plan(m, n, k, 1 if accumulate else 0, sms, ctypes.byref(s), ctypes.byref(t), ctypes.byref(r))
    return s.value, t.value, r.value


def pair_products(which) -> int:
    """Which products of many tokens may run on pairs of SMs (csrc/gemm_tc_pair.cu): a sum of 1 (plain products), 2 (the
    gated product) and 4 (the q/k/v product that finishes its heads); True: all (as at the start), False: none.
    Returns the setting before."""
    return lib().llmx_rt_pair_products(7 if which is True else 0 if which is False else int(which))


def heads_tile(m: int, heads: int, kv_heads: int, sms: int = 0) -> int:
    return lib().llmx_heads_tile(m, heads, kv_heads, sms)


def decode_schedule(n_requests: int, kv_heads: int, max_context: int, head_dim: int = 128, clusters=None):
    s, c = _i(), _i()
    table = None
    if clusters is not None:
        table = (ctypes.c_int * 17)(*[int(clusters.get(i, 0)) for i in range(17)])
    lib().llmx_decode_schedule(n_requests, kv_heads, max_context, head_dim, table, ctypes.byref(s), ctypes.byref(c))
    return s.value, c.value


def prefill_shape(n_requests: int, kv_heads: int, ratio: int, max_rows: int, max_context: int, window: int, sms: int = 148):
    t, s = _i(), _i()
    lib().llmx_prefill_shape(n_requests, kv_heads, ratio, max_rows, max_context, int(window or 0), sms, ctypes.byref(t), ctypes.byref(s))
    return t.value, s.value


def tiled_attention(heads: int, kv_heads: int, head_dim: int, page_size: int) -> int:
    """0: only the plain kernel takes this shape; 1: split-KV decode and warp-level prefill; 2: ... and tcgen05 prefill."""
    return lib().llmx_tiled_attention(heads, kv_heads, head_dim, page_size)


# ---- plans ------------------------------------------------------------------------------------------------------
class Plan:
    """Launch decisions of the native parts for one step shape (`llmx_plan_make`).  `room` > 0: for a step that
    is recorded and replayed; `fill` then follows the histories of the run at hand."""

    def __init__(self, model_handle, part_handles: Sequence[int], counts: Sequence[int], histories: Optional[Sequence[int]],
                 room: int = 0, typical_context: int = 0):
        n = len(counts)
        c = (ctypes.c_int * n)(*counts)
        h = (ctypes.c_int * n)(*histories) if histories is not None else None
        parts = (ctypes.c_void_p * len(part_handles))(*part_handles) if part_handles else None
        self.handle = lib().llmx_plan_make(model_handle, parts, len(part_handles), c, h, n, int(room), int(typical_context))
        if not self.handle:
            raise KernelError(last_error())
        self.ints = lib().llmx_plan_ints(self.handle)
        self.requests = n

    def fill(self, histories: Sequence[int], out: np.ndarray) -> None:
        if self.ints == 0:
            return
        h = (ctypes.c_int * self.requests)(*histories)
        assert out.dtype == np.int32 and out.size >= self.ints and out.flags["C_CONTIGUOUS"]
        check(lib().llmx_plan_fill(self.handle, h, out.ctypes.data), "plan")

    def force_prefill_shape(self, tiles: int, splits: int) -> None:
        lib().llmx_plan_force_prefill_shape(self.handle, tiles, splits)

    def force_decode(self, splits: int, chunk: int) -> None:
        lib().llmx_plan_force_decode(self.handle, splits, chunk)

    def describe(self) -> Optional[dict]:
        out = (ctypes.c_int * 8)()
        if not lib().llmx_plan_describe(self.handle, out):
            return None
        keys = ("small", "large", "splits", "chunk", "tiles", "prefill_splits", "rows_small", "rows_large")
        return dict(zip(keys, list(out)))

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h and _lib is not None:
            _lib.llmx_plan_free(h)


# ---- the cache's entries as the runtime sees them ------------------------------------------------------------
class CacheViews:
    """Where every cache entry's storage lies (`llmx_caches`); owns the TMA descriptors of the entries."""

    def __init__(self, entries: int):
        self.handle = lib().llmx_caches_create(entries)
        self._keep: List[torch.Tensor] = []

    def set_kv(self, entry: int, group: int, storage: torch.Tensor) -> None:
        pages, _, kv_heads, page_size, head_dim = storage.shape
        check(lib().llmx_caches_set_kv(self.handle, entry, group, storage.data_ptr(), code(storage.dtype), pages, kv_heads,
                                       page_size, head_dim), "cache entry")
        self._keep.append(storage)

    def set_state(self, entry: int, storage: torch.Tensor) -> None:
        per = storage[0].numel() * storage.element_size() if storage.shape[0] else 0
        check(lib().llmx_caches_set_state(self.handle, entry, storage.data_ptr(), storage.shape[0], per), "state entry")
        self._keep.append(storage)

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h and _lib is not None:
            _lib.llmx_caches_destroy(h)


# ---- kernel timing --------------------------------------------------------------------------------------------
def profile(on: bool) -> bool:
    return bool(lib().llmx_rt_profile(1 if on else 0))


def profile_results():
    out, k = [], 0
    name, ms, idle = ctypes.c_char_p(), _f(), _f()
    while lib().llmx_rt_profile_read(k, ctypes.byref(name), ctypes.byref(ms), ctypes.byref(idle)):
        out.append((name.value.decode(), ms.value, idle.value))
        k += 1
    return out
