"""Trace replay: feed given token ids through the engine step by step and write logits.

Reads one JSON object a line from a stream:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
runs each step through `Engine.step` (the step function generation uses),
writes `<out>/<step>.f32` (little-endian float32 [wanted, vocab]) when something
is wanted, frees the requests named in `end`, and prints `done <step>`.
It samples nothing and has no forward pass, cache or loader of its own.  The
reference's analogue handles one sequence (tools/model_logits.cpp:28-140); this
one replays any mix of requests.  With `--engine native` the same steps go through
the native engine (csrc/runtime/llmx_engine.h: its loader, its cache books, the same
model runtime and kernels).
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO

import torch

from .engine import Engine, EngineOptions, StepEntry


def replay(engine: Engine, lines: IO[str], out_dir: str, done: IO[str]) -> int:
    os.makedirs(out_dir, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in rec.get("entries", ())]
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                host = logits.to(torch.float32).cpu().contiguous()
                host.numpy().astype("<f4", copy=False).tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", ()):
            engine.end(rid)
        print(f"done {step}", file=done, flush=True)
    return 0


def replay_native(native, lines: IO[str], out_dir: str, done: IO[str]) -> int:
    """The same protocol over `NativeEngine.forward` (requests are named by numbers there)."""
    os.makedirs(out_dir, exist_ok=True)
    ids, next_id = {}, 1
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", ()):
            if e["id"] not in ids:
                ids[e["id"]], next_id = next_id, next_id + 1
            entries.append((ids[e["id"]], e["tokens"], e.get("want", ())))
        if entries:
            logits = native.forward(entries)
            if logits.shape[0]:
                logits.astype("<f4", copy=False).tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", ()):
            if rid in ids:
                native.end(ids.pop(rid))
        print(f"done {step}", file=done, flush=True)
    return 0


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="the most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--engine", choices=["python", "native"], default="python",
                    help="the Python engine (default) or the native one: the same model runtime and kernels either way")
    args = ap.parse_args(argv)
    if 64 % args.page_size and args.page_size % 64:
        ap.error("--page-size must divide 64 or be a multiple of it")
    kv_tokens = -(-args.max_tokens // args.page_size) * args.page_size
    if args.engine == "native":
        from ..native_engine import NativeEngine
        native = NativeEngine.load(args.model, dtype=args.dtype, kv_tokens=kv_tokens, page_size=args.page_size, max_requests=16,
                                   device=int(args.device.split(":")[1]) if ":" in args.device else 0)
        return replay_native(native, sys.stdin, args.out, sys.stdout)
    engine = Engine.from_dir(args.model, EngineOptions(dtype=args.dtype, kv_tokens=kv_tokens, page_size=args.page_size,
                                                       max_requests=16, device=args.device))
    return replay(engine, sys.stdin, args.out, sys.stdout)
