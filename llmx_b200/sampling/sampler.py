"""The sampler: per-request generators and penalties on the host, the draw on the device.

Each request has its own xorshift64 generator (src/inference/sampler.hpp:21-32) seeded from its
settings, and its own count of the tokens it has generated.  A draw uses one uniform number of
the request's generator, so what a request generates does not depend on what it was batched
with.  The logits never leave the device: `llmx_sample` picks the ids there and only those
are copied back.
"""
from __future__ import annotations

import ctypes
import struct
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..ops import _check, _cuda, _fn, _need, _ptr, _stream, register_signature
from .params import SamplingParams

_i, _p = ctypes.c_int, ctypes.c_void_p
register_signature("sampling", "llmx_sample", [_p, _i, _i, _p, _p, _i, _p])
register_signature("sampling", "llmx_penalize", [_p, _i, _p, _p, _p, _p, _p, _p, _i, _p])

_MASK = (1 << 64) - 1


class XorShift64:
    def __init__(self, seed: int = 0):
        self.state = 0x9E3779B97F4A7C15
        if seed:
            self.state = seed & _MASK

    def next(self) -> int:
        x = self.state
        x ^= (x << 13) & _MASK
        x ^= x >> 7
        x ^= (x << 17) & _MASK
        self.state = x
        return x

    def unit(self) -> float:
        """Uniform float in [0, 1): the top 24 bits."""
        return float(np.float32((self.next() >> 40) * (1.0 / 16777216.0)))


class RequestSampling:
    """One request's sampling state."""

    def __init__(self, params: SamplingParams, eos_id: int = -1):
        self.params = params
        self.rng = XorShift64(params.seed)
        self.counts: Dict[int, int] = {}
        self.masked = eos_id if params.ignore_eos else -1

    def saw(self, token: int) -> None:
        if self.params.penalized:
            self.counts[token] = self.counts.get(token, 0) + 1


_ROW = struct.Struct("<ffffii")


class PendingSample:
    """Ids that have been drawn on the device and are on their way to the host.  `ids` is the device tensor
    (int32 [rows]), which a next step may take as its input at once; `result()` waits for the copy."""
    __slots__ = ("ids", "_host", "_event")

    def __init__(self, ids: torch.Tensor, host: Optional[torch.Tensor], event):
        self.ids, self._host, self._event = ids, host, event

    def result(self) -> List[int]:
        if self._host is None:
            return []
        self._event.synchronize()
        return self._host.tolist()


def sample(logits: torch.Tensor, states: Sequence[RequestSampling]) -> List[int]:
    """One token per row of `logits` (float32 [rows, vocab] on the device), row i drawn for states[i]."""
    return sample_async(logits, states).result()


def sample_async(logits: torch.Tensor, states: Sequence[RequestSampling]) -> PendingSample:
    """As `sample`, but returns once the draw and the copy of the ids to the host are enqueued."""
    rows, vocab = logits.shape
    _cuda(logits)
    _need(logits.dtype is torch.float32 and len(states) == rows, "sample: float32 logits, one state per row")
    if rows == 0:
        return PendingSample(torch.empty(0, dtype=torch.int32, device=logits.device), None, None)
    dev = logits.device
    # Penalties first, in place: the logits are this step's own.
    items = [(r, t, c) for r, s in enumerate(states) if s.params.penalized for t, c in s.counts.items()]
    if items:
        arr = torch.tensor(items, dtype=torch.int32).t().contiguous().to(dev)
        pen = torch.tensor([[s.params.penalty, s.params.presence_penalty, s.params.frequency_penalty] for s in states],
                           dtype=torch.float32).t().contiguous().to(dev)
        _check(_fn("sampling", "llmx_penalize")(_ptr(logits), vocab, _ptr(arr[0]), _ptr(arr[1]), _ptr(arr[2]),
                                                _ptr(pen[0]), _ptr(pen[1]), _ptr(pen[2]), len(items), _stream()),
               "penalize")
    all_greedy = all(s.params.greedy for s in states)
    key = None
    if all_greedy:
        # Greedy rows draw nothing: their parameters are the same from step to step and stay on the device.
        key = (dev.index, tuple(s.masked for s in states))
    params = _greedy_params.get(key) if key is not None else None
    if params is None:
        raw = bytearray(_ROW.size * rows)
        for r, s in enumerate(states):
            p = s.params
            u = 0.0 if p.greedy else s.rng.unit()
            _ROW.pack_into(raw, r * _ROW.size, p.temp, p.top_p, p.min_p, u, p.top_k, s.masked)
        host = torch.empty(len(raw), dtype=torch.uint8, pin_memory=True)
        host.numpy()[:] = np.frombuffer(raw, dtype=np.uint8)
        params = host.to(dev, non_blocking=True)
        if key is not None:
            if len(_greedy_params) > 64:
                _greedy_params.clear()
            _greedy_params[key] = params
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    _check(_fn("sampling", "llmx_sample")(_ptr(logits), rows, vocab, _ptr(params), _ptr(out), 1 if all_greedy else 0,
                                          _stream()), "sample")
    host = torch.empty(rows, dtype=torch.int32, pin_memory=True)
    host.copy_(out, non_blocking=True)
    event = torch.cuda.Event()
    event.record()
    return PendingSample(out, host, event)


_greedy_params: Dict[tuple, torch.Tensor] = {}
