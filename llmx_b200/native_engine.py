"""A thin Python face of the native engine (csrc/runtime/llmx_engine.h): `load / add_request / step / forward`.

The native engine keeps the cache's bookkeeping, the step's metadata, the scheduler and the sampler's state in C++
and runs the same model runtime and kernels as `llmx_b200.engine.Engine`.  This module only converts arguments:

    e = NativeEngine.load(model_dir, dtype="bfloat16", kv_tokens=8192)       # files read by the native loader
    e = NativeEngine.over(engine)                                            # the weights a Python `Engine` has loaded
    rid = e.add_request([1, 2, 3], SamplingParams(max_tokens=8, temp=0))
    while not e.idle:
        for request, token, finished in e.step(): ...
    logits = e.forward([(7, [5, 17, 3], [0, 2])])                            # the low level: numpy [wanted, vocab]

Reference counterparts: `infer::load_model` (src/inference/load.hpp:74-94), `Model::forward / step`
(src/model/runtime.hpp:1278-1387), `infer::generate` (src/inference/generate.hpp:19-124).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import runtime
from .sampling.params import SamplingParams

_i, _p, _ll, _f, _ull = ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float, ctypes.c_ulonglong

ERR_REFUSED, ERR_CACHE, ERR_FILE, ERR_WEIGHTS, ERR_DEVICE, ERR_UNBOUND = 20001, 20002, 20003, 20004, 20005, 10010
FINISHED = {0: None, 1: "eos", 2: "length", 3: "cache"}


class NativeEngineError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(text)
        self.code = code


class CacheEntryDesc(ctypes.Structure):
    _fields_ = [("kind", _i), ("kv_heads", _i), ("head_dim", _i), ("window", _i), ("state_bytes", _ll)]


class EngineDesc(ctypes.Structure):
    _fields_ = [("vocab", _i), ("max_positions", _i), ("position_streams", _i), ("page_size", _i), ("kv_tokens", _ll),
                ("window_kv_tokens", _ll), ("max_requests", _i), ("kv_dtype", _i), ("entries", ctypes.POINTER(CacheEntryDesc)),
                ("n_entries", _i), ("eos_ids", ctypes.POINTER(_i)), ("n_eos", _i), ("max_batch_tokens", _i), ("max_queue", _i),
                ("reserve_prompt_only", _i), ("device", _i)]


class EngineOptionsC(ctypes.Structure):
    _fields_ = [("dtype", _i), ("kv_dtype", _i), ("page_size", _i), ("kv_tokens", _ll), ("window_kv_tokens", _ll),
                ("max_requests", _i), ("max_batch_tokens", _i), ("max_queue", _i), ("reserve_prompt_only", _i), ("invariant", _i),
                ("device", _i), ("kernel_dir", ctypes.c_char_p)]


class SamplingC(ctypes.Structure):
    _fields_ = [("max_tokens", _i), ("temp", _f), ("top_k", _i), ("top_p", _f), ("min_p", _f), ("penalty", _f),
                ("presence_penalty", _f), ("frequency_penalty", _f), ("seed", _ull), ("ignore_eos", _i),
                ("stop_ids", ctypes.POINTER(_i)), ("n_stop", _i)]


class EntryC(ctypes.Structure):
    _fields_ = [("request", _ll), ("tokens", ctypes.POINTER(_i)), ("n_tokens", _i), ("want", ctypes.POINTER(_i)), ("n_want", _i)]


class StepResultC(ctypes.Structure):
    _fields_ = [("request", _ll), ("token", _i), ("finished", _i)]


class PlannedEntryC(ctypes.Structure):
    _fields_ = [("request", _ll), ("n_tokens", _i), ("first_token", _i), ("want_last", _i)]


_SIGNATURES = {
    "llmx_engine_create": (_p, [_p, ctypes.POINTER(EngineDesc)]),
    "llmx_engine_load": (_p, [ctypes.c_char_p, ctypes.POINTER(EngineOptionsC)]),
    "llmx_engine_destroy": (None, [_p]),
    "llmx_engine_last_error": (ctypes.c_char_p, []),
    "llmx_engine_last_code": (_i, []),
    "llmx_engine_forward": (_i, [_p, ctypes.POINTER(EntryC), _i, _p, _p]),
    "llmx_engine_end": (_i, [_p, _ll]),
    "llmx_engine_truncate": (_i, [_p, _ll, _i]),
    "llmx_engine_length": (_i, [_p, _ll]),
    "llmx_engine_add_request": (_ll, [_p, ctypes.POINTER(_i), _i, ctypes.POINTER(SamplingC)]),
    "llmx_engine_step": (_i, [_p, ctypes.POINTER(StepResultC), _i]),
    "llmx_engine_idle": (_i, [_p]),
    "llmx_engine_plan": (_i, [_p, ctypes.POINTER(PlannedEntryC), _i]),
    "llmx_engine_book": (_i, [_p, ctypes.POINTER(_i), _i, ctypes.POINTER(StepResultC), _i]),
    "llmx_engine_last_logits": (_i, [_p, _p, _p]),
    "llmx_engine_output": (_i, [_p, _ll, ctypes.POINTER(_i), _i, ctypes.POINTER(_i)]),
    "llmx_engine_forget": (_i, [_p, _ll]),
    "llmx_engine_groups": (_i, [_p]),
    "llmx_engine_pages": (_i, [_p, _i, ctypes.POINTER(_ll), ctypes.POINTER(_ll)]),
    "llmx_engine_held_pages": (_i, [_p, _ll, _i]),
    "llmx_engine_check": (_i, [_p]),
    "llmx_engine_preemptions": (_ll, [_p]),
    "llmx_engine_steps": (_ll, [_p]),
    "llmx_engine_replays": (_ll, [_p]),
    "llmx_engine_record_steps": (None, [_p, _i]),
    "llmx_engine_last_h2d_bytes": (_ll, [_p]),
    "llmx_engine_vocab": (_i, [_p]),
    "llmx_engine_max_positions": (_i, [_p]),
}
_ready = False


def _lib():
    global _ready
    rt = runtime.lib()
    if not _ready:
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(rt, name)
            fn.restype, fn.argtypes = restype, argtypes
        _ready = True
    return rt


def _error(code: int) -> NativeEngineError:
    return NativeEngineError(int(code), (_lib().llmx_engine_last_error() or b"").decode("utf-8", "replace") or f"error {code}")


def _ints(values: Sequence[int]):
    arr = (_i * max(len(values), 1))(*[int(v) for v in values])
    return arr


def _dtype_code(name: Optional[str]) -> int:
    if name is None:
        return -1
    if name in ("bfloat16", "bf16"):
        return runtime.BF16
    if name in ("float32", "f32", "fp32"):
        return runtime.F32
    raise ValueError(f"dtype {name!r} is not one the engine takes (bfloat16, float32)")


def _sampling(params: SamplingParams):
    stops = _ints(params.stop_token_ids)
    s = SamplingC(params.max_tokens, params.temp, params.top_k, params.top_p, params.min_p, params.penalty,
                  params.presence_penalty, params.frequency_penalty, params.seed, 1 if params.ignore_eos else 0,
                  ctypes.cast(stops, ctypes.POINTER(_i)), len(params.stop_token_ids))
    return s, stops


class NativeEngine:
    def __init__(self, handle: int, keep=()):
        if not handle:
            raise _error(_lib().llmx_engine_last_code() or ERR_REFUSED)
        self._h = ctypes.c_void_p(handle)
        self._keep = keep                     # what the native engine points into and does not own
        self.vocab = _lib().llmx_engine_vocab(self._h)
        self.max_positions = _lib().llmx_engine_max_positions(self._h)

    # -- construction -------------------------------------------------------------------------------------------
    @classmethod
    def over(cls, engine, *, kv_tokens: Optional[int] = None, page_size: Optional[int] = None, max_requests: Optional[int] = None,
             ubatch: int = 2048, reserve: str = "full", kv_dtype: Optional[str] = None) -> "NativeEngine":
        """A native engine over the model a Python `Engine` has loaded (the weights are shared; the cache is its own)."""
        from .cache.manager import KVSpec, StateSpec
        model, opt = engine.model, engine.options
        handle = model.native
        if handle is None:
            raise ValueError("the model has parts written in Python; the native engine runs models that are native throughout")
        specs = model.cache_entry_specs()
        entries = (CacheEntryDesc * max(len(specs), 1))()
        for i, s in enumerate(specs):
            if isinstance(s, KVSpec):
                entries[i] = CacheEntryDesc(1, s.kv_heads, s.head_dim, int(s.window or 0), 0)
            elif isinstance(s, StateSpec):
                import torch
                size = int(np.prod(s.shape)) * torch.empty(0, dtype=getattr(torch, s.dtype)).element_size()
                entries[i] = CacheEntryDesc(2, 0, 0, 0, size)
            else:
                entries[i] = CacheEntryDesc(0, 0, 0, 0, 0)
        eos = _ints(model.eos_ids)
        kv = _dtype_code(kv_dtype or opt.kv_dtype or opt.dtype)
        tokens = int(kv_tokens if kv_tokens is not None else opt.kv_tokens)
        if tokens > opt.kv_tokens and any(isinstance(s, KVSpec) and s.window is None for s in specs):
            raise ValueError("the model's position tables were made for the Python engine's kv_tokens; ask for no more")
        import torch
        desc = EngineDesc(model.vocab_size, model.max_positions, model.position_streams, int(page_size or opt.page_size), tokens,
                          int(opt.window_kv_tokens or 0), int(max_requests or opt.max_requests), kv, entries, len(specs),
                          ctypes.cast(eos, ctypes.POINTER(_i)), len(model.eos_ids), int(ubatch), 0, 1 if reserve == "prompt" else 0,
                          torch.device(opt.device).index or 0)
        if reserve not in ("full", "prompt"):
            raise ValueError("reserve must be 'full' or 'prompt'")
        return cls(_lib().llmx_engine_create(ctypes.c_void_p(handle), ctypes.byref(desc)), keep=(engine, entries, eos))

    @classmethod
    def books(cls, entries: Sequence[Tuple[int, int, int]], *, page_size: int = 16, kv_tokens: int = 8192,
              window_kv_tokens: int = 0, max_requests: int = 16, ubatch: int = 512, reserve: str = "full", max_queue: int = 0,
              vocab: int = 1 << 30, max_positions: int = 1 << 30, eos_ids: Sequence[int] = ()) -> "NativeEngine":
        """The native engine's books alone (no model, no device): the scheduler's decisions and the cache's pages, for a
        caller that supplies the tokens (`plan`, `book`).  `entries`: (kv_heads, head_dim, window) per cache entry."""
        if reserve not in ("full", "prompt"):
            raise ValueError("reserve must be 'full' or 'prompt'")
        arr = (CacheEntryDesc * max(len(entries), 1))()
        for i, (kvh, d, w) in enumerate(entries):
            arr[i] = CacheEntryDesc(1, int(kvh), int(d), int(w or 0), 0)
        eos = _ints(eos_ids)
        desc = EngineDesc(int(vocab), int(max_positions), 1, int(page_size), int(kv_tokens), int(window_kv_tokens), int(max_requests),
                          runtime.BF16, arr, len(entries), ctypes.cast(eos, ctypes.POINTER(_i)), len(eos_ids), int(ubatch),
                          int(max_queue), 1 if reserve == "prompt" else 0, -1)
        return cls(_lib().llmx_engine_create(None, ctypes.byref(desc)), keep=(arr, eos))

    @staticmethod
    def _options(dtype, kv_dtype, page_size, kv_tokens, window_kv_tokens, max_requests, ubatch, reserve, invariant, device):
        if reserve not in ("full", "prompt"):
            raise ValueError("reserve must be 'full' or 'prompt'")
        return EngineOptionsC(_dtype_code(dtype), _dtype_code(kv_dtype), int(page_size), int(kv_tokens), int(window_kv_tokens or 0),
                              int(max_requests), int(ubatch), 0, 1 if reserve == "prompt" else 0, 1 if invariant else 0, int(device), None)

    @classmethod
    def load(cls, model_dir: str, *, dtype: str = "bfloat16", kv_dtype: Optional[str] = None, page_size: int = 16,
             kv_tokens: int = 8192, window_kv_tokens: Optional[int] = None, max_requests: int = 16, ubatch: int = 2048,
             reserve: str = "full", invariant: bool = False, device: int = 0) -> "NativeEngine":
        """config.json and the safetensors files of `model_dir`, read by the native loader."""
        opts = cls._options(dtype, kv_dtype, page_size, kv_tokens, window_kv_tokens, max_requests, ubatch, reserve, invariant, device)
        return cls(_lib().llmx_engine_load(str(model_dir).encode(), ctypes.byref(opts)))

    def close(self) -> None:
        if self._h:
            _lib().llmx_engine_destroy(self._h)
            self._h = None
            self._keep = ()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- calls that may find a kernel library not loaded yet: load it and call again ------------------------------
    def _call(self, fn, *args):
        for _ in range(16):
            status = fn(*args)
            if status in (ERR_UNBOUND, -ERR_UNBOUND):
                if not runtime.bind_missing():
                    raise _error(ERR_UNBOUND)
                continue
            return status
        raise _error(ERR_UNBOUND)

    # -- the low level ---------------------------------------------------------------------------------------------
    def forward(self, entries: Sequence[Tuple[int, Sequence[int], Sequence[int]]]) -> np.ndarray:
        """One batch of (request, its next tokens, wanted places); float32 logits [wanted, vocab]."""
        keep, raw = [], (EntryC * max(len(entries), 1))()
        wanted = 0
        for k, (request, tokens, want) in enumerate(entries):
            t, w = _ints(tokens), _ints(want)
            keep += [t, w]
            raw[k] = EntryC(int(request), ctypes.cast(t, ctypes.POINTER(_i)), len(tokens), ctypes.cast(w, ctypes.POINTER(_i)), len(want))
            wanted += len(want)
        out = np.empty((wanted, self.vocab), dtype=np.float32)
        status = self._call(_lib().llmx_engine_forward, self._h, raw, len(entries), out.ctypes.data_as(_p), None)
        if status:
            raise _error(status)
        return out

    def end(self, request: int) -> None:
        _lib().llmx_engine_end(self._h, int(request))

    def truncate(self, request: int, length: int) -> None:
        status = _lib().llmx_engine_truncate(self._h, int(request), int(length))
        if status:
            raise _error(status)

    def length(self, request: int) -> int:
        return _lib().llmx_engine_length(self._h, int(request))

    # -- generation ------------------------------------------------------------------------------------------------
    def add_request(self, ids: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        s, stops = _sampling(params or SamplingParams())
        arr = _ints(ids)
        rid = _lib().llmx_engine_add_request(self._h, ctypes.cast(arr, ctypes.POINTER(_i)), len(ids), ctypes.byref(s))
        if rid < 0:
            raise _error(-rid)
        return int(rid)

    def step(self) -> List[Tuple[int, int, Optional[str]]]:
        """Plan a step, run it, draw and book: [(request, token or -1, None | "eos" | "length" | "cache")]."""
        raw = (StepResultC * 1024)()
        n = self._call(_lib().llmx_engine_step, self._h, raw, 1024)
        if n < 0:
            raise _error(-n)
        return [(int(raw[k].request), int(raw[k].token), FINISHED[raw[k].finished]) for k in range(n)]

    def plan(self) -> List[Tuple[int, int, int, bool]]:
        """The first half of `step`: plan, reserve pages and (with a model) run.  [(request, tokens, first token, wants a
        token)]; an empty list when nothing is to run."""
        raw = (PlannedEntryC * 4096)()
        n = self._call(_lib().llmx_engine_plan, self._h, raw, 4096)
        if n < 0:
            raise _error(-n)
        return [(int(raw[k].request), int(raw[k].n_tokens), int(raw[k].first_token), bool(raw[k].want_last)) for k in range(n)]

    def book(self, drawn: Sequence[int]) -> List[Tuple[int, int, Optional[str]]]:
        """The second half: one token for every planned entry that wanted one, in order."""
        raw = (StepResultC * 4096)()
        arr = _ints(drawn)
        n = _lib().llmx_engine_book(self._h, ctypes.cast(arr, ctypes.POINTER(_i)), len(drawn), raw, 4096)
        if n < 0:
            raise _error(-n)
        return [(int(raw[k].request), int(raw[k].token), FINISHED[raw[k].finished]) for k in range(n)]

    def last_logits(self) -> np.ndarray:
        """The logits of the step that ran last, [wanted, vocab]."""
        n = _lib().llmx_engine_last_logits(self._h, None, None)
        if n < 0:
            raise _error(-n)
        out = np.empty((n, self.vocab), dtype=np.float32)
        if n and _lib().llmx_engine_last_logits(self._h, out.ctypes.data_as(_p), None) < 0:
            raise _error(ERR_DEVICE)
        return out

    @property
    def idle(self) -> bool:
        return bool(_lib().llmx_engine_idle(self._h))

    def output(self, request: int) -> Tuple[List[int], Optional[str]]:
        buf, fin = (_i * self.max_positions)(), _i(0)
        n = _lib().llmx_engine_output(self._h, int(request), buf, self.max_positions, ctypes.byref(fin))
        if n < 0:
            raise _error(-n)
        return list(buf[:n]), FINISHED[fin.value]

    def forget(self, request: int) -> None:
        _lib().llmx_engine_forget(self._h, int(request))

    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[Tuple[List[int], Optional[str]]]:
        """A reply for every prompt: [(tokens, finish reason)] in the prompts' order."""
        plist = [params or SamplingParams()] * len(prompts) if params is None or isinstance(params, SamplingParams) else list(params)
        ids = [self.add_request(p, q) for p, q in zip(prompts, plist)]
        while not self.idle:
            self.step()
        out = [self.output(r) for r in ids]
        for r in ids:
            self.forget(r)
        return out

    # -- accounting ------------------------------------------------------------------------------------------------
    def pages(self) -> List[Tuple[int, int]]:
        """(total, free) pages of every cache group."""
        out = []
        for g in range(_lib().llmx_engine_groups(self._h)):
            total, free = _ll(0), _ll(0)
            _lib().llmx_engine_pages(self._h, g, ctypes.byref(total), ctypes.byref(free))
            out.append((total.value, free.value))
        return out

    def held_pages(self, request: int, group: int = 0) -> int:
        return _lib().llmx_engine_held_pages(self._h, int(request), group)

    def check(self) -> None:
        status = _lib().llmx_engine_check(self._h)
        if status:
            raise AssertionError(str(_error(status)))

    @property
    def preemptions(self) -> int:
        return int(_lib().llmx_engine_preemptions(self._h))

    @property
    def steps(self) -> int:
        return int(_lib().llmx_engine_steps(self._h))

    @property
    def replays(self) -> int:
        """Steps that replayed a recorded (CUDA graph) step."""
        return int(_lib().llmx_engine_replays(self._h))

    def record_steps(self, on: bool) -> None:
        """Whether step shapes that keep coming are recorded as CUDA graphs (on at the start)."""
        _lib().llmx_engine_record_steps(self._h, 1 if on else 0)

    @property
    def last_h2d_bytes(self) -> int:
        return int(_lib().llmx_engine_last_h2d_bytes(self._h))
