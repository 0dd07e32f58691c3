"""Helpers of the engine tests: traces in the replay format, and running them.

A trace is a list of steps `{"step", "entries": [{"id", "tokens", "want"}], "end"}`, the format
`bin/trace_run` reads.  The builders below make the four ways of cutting the same requests that
the tests compare: whole, most of it then the last tokens one by one, portions of changing size,
and a mix of up to four live requests with pages that are used again.
"""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, List, Sequence, Tuple

import numpy as np

import plain_qwen3 as plain

PORTIONS = [7, 2, 13, 3, 2, 29, 5, 2, 17, 64, 3, 11]


def random_ids(vocab: int, n: int, seed: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def trace_whole(requests: Dict[str, List[int]]) -> List[dict]:
    steps = []
    for i, (rid, ids) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]})
    return steps


def trace_tail_decoded(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    steps, n = [], 0
    for rid, ids in requests.items():
        head = max(len(ids) - tail, 0)
        if head:
            steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []})
            n += 1
        for t in range(head, len(ids)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [ids[t]], "want": [0]}],
                          "end": [rid] if t == len(ids) - 1 else []})
            n += 1
    return steps


def trace_portions(requests: Dict[str, List[int]], portions: Sequence[int] = PORTIONS) -> List[dict]:
    steps, n, k = [], 0, 0
    for rid, ids in requests.items():
        at = 0
        while at < len(ids):
            p = min(portions[k % len(portions)], len(ids) - at)
            k += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[at:at + p], "want": list(range(p))}],
                          "end": [rid] if at + p == len(ids) else []})
            at += p
            n += 1
    return steps


def trace_mixed(requests: Dict[str, List[int]], tail: int = 12, live_max: int = 4,
                portions: Sequence[int] = PORTIONS) -> List[dict]:
    """Up to `live_max` live requests: each feeds its prompt in portions of changing size, then its last
    `tail` tokens one by one, beside whatever the others are doing; a finished request makes room for the
    next, so with a tight pool its pages are used again.  Every third step one live request sits out."""
    waiting = list(requests.items())
    live: List[list] = []          # [rid, ids, at]
    steps, n, k = [], 0, 0
    while waiting or live:
        while waiting and len(live) < live_max:
            rid, ids = waiting.pop(0)
            live.append([rid, ids, 0])
        entries, ended = [], []
        skip = live[n % len(live)][0] if (n % 3 == 2 and len(live) > 1) else None
        for item in live:
            rid, ids, at = item
            if rid == skip:
                continue
            head = max(len(ids) - tail, 0)
            if at < head:
                p = min(portions[k % len(portions)], head - at)
                k += 1
            else:
                p = 1
            entries.append({"id": rid, "tokens": ids[at:at + p], "want": list(range(p))})
            item[2] = at + p
            if item[2] == len(ids):
                ended.append(rid)
        live = [it for it in live if it[0] not in ended]
        steps.append({"step": n, "entries": entries, "end": ended})
        n += 1
    return steps


def tokens_needed(steps: List[dict], page: int = 64) -> int:
    """The most tokens live requests hold at any time, each request's count rounded up to `page`."""
    held: Dict[str, int] = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-v // page) * page for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


def run_trace(engine, steps: List[dict], record: bool = False) -> Dict[Tuple[str, int], np.ndarray]:
    """Drive Engine.step with a trace; returns {(request, position): logits row}."""
    from llmx_b200.engine import StepEntry
    out: Dict[Tuple[str, int], np.ndarray] = {}
    at: Dict[str, int] = {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        logits = engine.step(entries, record=record)
        rows = None if logits is None else logits.float().cpu().numpy()
        k = 0
        for e in s["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = rows[k]
                k += 1
            at[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            engine.end(rid)
            at.pop(rid, None)
    return out


def read_trace_output(steps: List[dict], out_dir: str, vocab: int) -> Dict[Tuple[str, int], np.ndarray]:
    """The same mapping from the files bin/trace_run wrote."""
    out: Dict[Tuple[str, int], np.ndarray] = {}
    at: Dict[str, int] = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        rows = None
        if wanted:
            rows = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(wanted, vocab)
        k = 0
        for e in s["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = rows[k]
                k += 1
            at[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            at.pop(rid, None)
    return out


@functools.lru_cache(maxsize=None)
def _folder(model_dir: str):
    return plain.load_folder(model_dir)


_ref_cache: Dict[tuple, np.ndarray] = {}


def reference_logits(model_dir: str, ids: Sequence[int], bf16: bool, cache: str = "same") -> np.ndarray:
    """Logits [len(ids), vocab] of the plain implementation; with `bf16`, rounding what that path rounds.
    `cache`: "same" (the cache has the path's type), "float32" or "bfloat16" (a cache type of its own)."""
    key = (model_dir, tuple(ids), bf16, cache)
    if key not in _ref_cache:
        cfg, w = _folder(model_dir)
        cache_round = {"same": "same", "float32": None, "bfloat16": plain.round_bf16}[cache]
        _ref_cache[key] = plain.forward(cfg, w, list(ids), act_round=plain.round_bf16 if bf16 else None, cache_round=cache_round)
    return _ref_cache[key]


def compare(got: Dict[Tuple[str, int], np.ndarray], requests: Dict[str, List[int]], model_dir: str, bf16: bool,
            cache: str = "same"):
    """(largest absolute difference, logit scale, where) over every wanted position."""
    worst, where, scale = 0.0, None, 0.0
    for rid, ids in requests.items():
        ref = reference_logits(model_dir, ids, bf16, cache)
        scale = max(scale, float(np.abs(ref).max()))
        for p in range(len(ids)):
            if (rid, p) not in got:
                continue
            d = float(np.abs(got[(rid, p)] - ref[p]).max())
            if not np.isfinite(d):
                return float("inf"), scale, (rid, p)
            if d > worst:
                worst, where = d, (rid, p)
    return worst, scale, where
