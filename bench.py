#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B sizes, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context C]

A "step" is one decode step: every live request brings one token.  The default run has the layer
sizes of Qwen3-8B (36 layers unless --layers says otherwise), a batch of 8 and a context of 8,192
tokens per request.  One JSON line is printed:

  value        decoded tokens a second, the K steps timed on the device with CUDA events
  e2e          the same through the Python entry point, `LLM.generate`: prompts of the context's length as host
               token ids in (it prefills them itself), sampled ids out; every step copies its metadata from
               pinned host memory and reads the drawn ids back; timed on the host between two tokens K steps apart
  prefill      a 2,048-token prompt from an empty cache: tokens a second and the fraction of the
               measured bf16 peak its flops reach
  roofline     the bytes a decode step must read (every weight once, the cache of the live requests)
               divided by its time, against the measured copy bandwidth
  points       decode tokens a second at batch 1 and batch 64 (mean and sd over three timed regions, and the fraction
               of the copy bandwidth), then the architecture's other published sizes: Qwen3-0.6B (decode at batch 64,
               context 4,096; a 2,048-token prompt) and Qwen3-32B (decode at batch 1, 8, 32, context 4,096; a
               2,048-token prompt), each with its roofline fraction
  repeats      mean and sd of the headline over three timed regions of K steps (`value` is the first)

For `value` and `points` the histories of the decoding requests are synthetic cache contents (pages taken and
filled with random values): what a decode step costs depends on how much it reads, not on what it reads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
                intermediate_size=12288, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=40960)


# Other published sizes of the same architecture (other widths and depths), for `--size`.
SIZES = {
    "8b": {},
    "0.6b": dict(num_hidden_layers=28, hidden_size=1024, intermediate_size=3072, num_attention_heads=16,
                 num_key_value_heads=8, tie_word_embeddings=True),
    "14b": dict(num_hidden_layers=40, hidden_size=5120, intermediate_size=17408, num_attention_heads=40,
                num_key_value_heads=8),          # five query heads a kv head
    "32b": dict(num_hidden_layers=64, hidden_size=5120, intermediate_size=25600, num_attention_heads=64,
                num_key_value_heads=8),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = os.path.join(tempfile.gettempdir(), f"llmx_clocks_{os.getpid()}.csv")

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        os.remove(self.path)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    """The unmodified reference, built with its own CMake and timed by its own `llmx bench` on the same
    configuration (baseline/reference_arm.py); nothing of llmx_b200 is imported on this path."""
    from baseline import reference_arm as arm
    raw = dict(QWEN3_8B)
    raw.update(SIZES[args.size])
    if args.layers is not None:
        raw["num_hidden_layers"] = args.layers
    raw["torch_dtype"] = "bfloat16"
    return arm.main(args, raw, args.size)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--size", choices=sorted(SIZES), default="8b", help="layer sizes: Qwen3-8B (the default), 0.6B, 14B or 32B")
    ap.add_argument("--profile", action="store_true",
                    help="with --only: also the device time by kernel of one plain (unrecorded) step, and the host's time for it")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--only", choices=["decode", "prefill", "sample"], default=None,
                    help="run one part only (for profiling); the line then holds only that part")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built in this engine")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import gc
    import statistics
    import torch
    from llmx_b200 import ops, ops_tc
    from llmx_b200.config import Qwen3Config
    from llmx_b200.engine import Engine, EngineOptions, StepEntry
    from llmx_b200.engine.decode_loop import DecodeSession
    from llmx_b200.sampling import RequestSampling, SamplingParams, sample

    pk = peaks()
    page = 16
    torch.cuda.set_device(0)
    host_gen = torch.Generator()
    host_gen.manual_seed(2)

    class Bench:
        """One model size on the device: its engine, and the timed runs over it."""

        def __init__(self, size, layers, batches, context, prefill_tokens, steps, warmup):
            raw = dict(QWEN3_8B)
            raw.update(SIZES[size])
            self.size, self.model_layers = size, raw["num_hidden_layers"]
            self.layers = layers if layers is not None else self.model_layers
            raw["num_hidden_layers"] = self.layers
            self.cfg = cfg = Qwen3Config.from_dict(raw)
            self.context, self.prefill_tokens = context, prefill_tokens
            E, F, Q, KV, V, L = cfg.hidden_size, cfg.intermediate_size, cfg.q_width, cfg.kv_width, cfg.vocab_size, self.layers
            # bytes a decode step must read: every weight once (a tied head reads the embedding table as its weight: the
            # same V * E bytes), the batch's embedding rows and the cache of the live requests
            self.weight_bytes = 2 * (L * ((Q + 2 * KV) * E + E * Q + 2 * F * E + E * F) + V * E) + 4 * (L * (2 * E + 2 * cfg.head_dim) + E)
            self.kv_bytes_per_token = L * 2 * KV * 2
            resident = 2 * (L * (E * (Q + 2 * KV) + Q * E + 3 * E * F) + V * E * (1 if cfg.tie_word_embeddings else 2))
            head_start = -(-context // 2048) * (max(batches, default=1) - 1)          # see run_generate
            per_request = -(-(context + 3 * steps + max(warmup, 8) + head_start + 64) // page) * page      # three timed regions (REPEATS)
            room = torch.cuda.get_device_properties(0).total_memory * 0.9 - resident - (8 << 30)
            self.batches = [b for b in batches if b * per_request * self.kv_bytes_per_token <= room]
            self.left_out = [b for b in batches if b not in self.batches]
            if not self.batches and batches:
                raise RuntimeError(f"a cache of {min(batches)} x {per_request} tokens does not fit beside the weights "
                                   f"({resident / 1e9:.0f} GB); give a smaller --batch, --context or --layers")
            max_batch = max(self.batches, default=1)
            kv_tokens = max(max_batch * per_request if self.batches else 0, prefill_tokens + page)
            self.engine = Engine.from_config(cfg, seed=0, options=EngineOptions(dtype="bfloat16", kv_tokens=kv_tokens, page_size=page,
                                                                                max_requests=max_batch, record_after=2))
            gen = torch.Generator(device="cuda")
            gen.manual_seed(1)
            for g in self.engine.cache.groups:          # synthetic histories: random keys and values
                for layer in range(g.storage.shape[0]):
                    g.storage[layer].normal_(0.0, 1.0, generator=gen)

        def close(self):
            self.engine = None
            gc.collect()
            torch.cuda.synchronize()
            torch.cuda.empty_cache()

        def ids(self, n):
            return torch.randint(0, self.cfg.vocab_size, (n,), generator=host_gen).tolist()

        def decode_bytes(self, batch):
            return self.weight_bytes + batch * self.cfg.hidden_size * 2 + batch * self.context * self.kv_bytes_per_token

        def hbm_frac(self, batch, ms):
            return self.decode_bytes(batch) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]

        def run_decode(self, batch, steps, warmup, repeats=1):
            """ms a step of `repeats` timed regions of `steps` decode steps each, for `batch` requests at `context`
            tokens; the launches of the first region; the bytes a step copies to the device."""
            engine = self.engine
            rids = [("bench", batch, i) for i in range(batch)]
            for rid in rids:                                    # take pages for the history without running it
                rc = engine.cache.new_request(rid)
                rc.prepare(self.context)
                rc.commit()
            session = DecodeSession(engine, rids)
            tokens = self.ids(batch)
            try:
                for _ in range(warmup):
                    session.step(tokens)
                torch.cuda.synchronize()
                times, launches = [], None
                for _ in range(repeats):
                    launches0 = ops.launch_count()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(steps):
                        session.step(tokens)
                    e1.record()
                    torch.cuda.synchronize()
                    times.append(e0.elapsed_time(e1) / steps)
                    launches = launches if launches is not None else ops.launch_count() - launches0
                h2d = session.h2d_bytes_per_step
            finally:
                session.close()
                for rid in rids:
                    engine.end(rid)
            return times, launches, h2d

        def run_generate(self, batch, steps, warmup):
            """The same decode rate through the Python entry point, `LLM.generate`: host token ids in (prompts of
            `context` tokens, which it prefills itself), sampled ids out.  Every step copies its metadata from pinned
            host memory and reads the drawn ids back; the clock runs between the callbacks of two tokens of the
            batch's last request, `steps` steps apart, after `warmup` decode steps."""
            from llmx_b200.engine.generate import LLM
            llm = LLM(self.engine, ubatch=2048, max_seqs=batch)
            prompts = [self.ids(self.context) for _ in range(batch)]
            seen, marks = [0], {}

            def on_token(i, token):
                if i == batch - 1:
                    seen[0] += 1
                    if seen[0] in (warmup + 1, warmup + 1 + steps):
                        marks[seen[0]] = time.perf_counter()
            # The requests' prompts end one after the other, so the first request decodes `head_start` steps before
            # the last one starts; all must still be decoding when the last one's timed tokens are drawn.
            head_start = -(-self.context // 2048) * (batch - 1)
            llm.generate(prompts, SamplingParams(max_tokens=head_start + warmup + steps + 4, temp=0.0, top_k=0, top_p=1.0,
                                                 ignore_eos=True), on_token)
            ms = (marks[warmup + 1 + steps] - marks[warmup + 1]) * 1e3 / steps
            h2d = max((rec.total * 4 for (b, _), rec in self.engine.decode_recordings.items() if b == batch), default=0)
            return batch * 1e3 / ms, ms, h2d

        def run_native(self, batch, steps, warmup):
            """The same decode rate through the native engine (csrc/runtime/llmx_engine.h: cache bookkeeping, scheduler,
            step metadata and sampler state in C++) over the same weights: `add_request` with host token ids, `step`
            until the last request has drawn its timed tokens.  Every step copies its metadata from pinned host memory,
            draws on the device and reads the ids back before the next is planned."""
            from llmx_b200.native_engine import NativeEngine
            head_start = -(-self.context // 2048) * (batch - 1)
            budget = head_start + warmup + steps + 4
            tokens = batch * (self.context + budget + 64)
            native = NativeEngine.over(self.engine, kv_tokens=min(tokens, self.engine.options.kv_tokens), ubatch=2048, max_requests=batch)
            try:
                params = SamplingParams(max_tokens=budget, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True)
                ids = [native.add_request(self.ids(self.context), params) for _ in range(batch)]
                seen, marks, h2d = 0, {}, 0
                while not native.idle:
                    for rid, token, _ in native.step():
                        if rid == ids[-1] and token >= 0:
                            seen += 1
                            if seen in (warmup + 1, warmup + 1 + steps):
                                marks[seen] = time.perf_counter()
                                h2d = native.last_h2d_bytes          # of a step of the whole batch
                ms = (marks[warmup + 1 + steps] - marks[warmup + 1]) * 1e3 / steps
                return batch * 1e3 / ms, ms, h2d, native.replays
            finally:
                native.close()

        def profile_plain_step(self, entries, what):
            """One plain (unrecorded) step of these entries: the host's time to enqueue it (the device idle, then
            free to run ahead) and the device time by kernel entry point (`ops.kernel_times`; printed to stderr)."""
            engine = self.engine
            ids = [e.request_id for e in entries]

            def undo():
                for e in entries:
                    rc = engine.cache.live[e.request_id]
                    if rc.length == len(e.tokens):
                        engine.end(e.request_id)
                    else:
                        engine.truncate(e.request_id, rc.length - len(e.tokens))
            for _ in range(3):
                engine.step(entries)
                undo()
            torch.cuda.synchronize()
            host = []
            for _ in range(5):
                t0 = time.perf_counter()
                engine.step(entries)
                host.append((time.perf_counter() - t0) * 1e3)
                torch.cuda.synchronize()
                undo()
            launches0 = ops.launch_count()
            with ops.kernel_times() as times:
                engine.step(entries)
            kernels = ops.launch_count() - launches0
            for rid in ids:
                engine.end(rid)
            for l in times.lines(what):
                print(l, file=sys.stderr)
            host.sort()
            return {"host_ms_per_plain_step": round(host[len(host) // 2], 4), "kernels": kernels,
                    "host_us_per_kernel": round(host[len(host) // 2] * 1e3 / max(kernels, 1), 2),
                    "device_ms_by_kernel": {k: round(v[1], 4) for k, v in times.by_function.items()},
                    "device_ms": round(times.total_ms, 4)}

        def run_prefill(self, reps, warmup):
            """(tokens a second, ms: mean and sd over `reps` prompts from an empty cache, fraction of the bf16 peak)."""
            cfg, T, L = self.cfg, self.prefill_tokens, self.layers
            E, F, Q, KV, V = cfg.hidden_size, cfg.intermediate_size, cfg.q_width, cfg.kv_width, cfg.vocab_size
            prompt = self.ids(T)
            times = []
            for i in range(warmup + reps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                self.engine.step([StepEntry("prefill", prompt, [T - 1])], record=True)
                e1.record()
                torch.cuda.synchronize()
                self.engine.end("prefill")
                if i >= warmup:
                    times.append(e0.elapsed_time(e1))
            ms = sum(times) / len(times)
            sd = statistics.stdev(times) if len(times) > 1 else 0.0
            flops = L * (2 * T * E * (Q + 2 * KV) + 2 * T * Q * E + 2 * T * E * 2 * F + 2 * T * F * E) \
                + L * 2 * cfg.num_attention_heads * cfg.head_dim * T * T + 2 * V * E
            return T * 1e3 / ms, ms, sd, flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"]

    def rate(batch, ms_list):
        """(mean tokens a second, its standard deviation over the repeats)."""
        rates = [batch * 1e3 / ms for ms in ms_list]
        return sum(rates) / len(rates), (statistics.stdev(rates) if len(rates) > 1 else 0.0)

    if args.only == "sample":
        # The sampling kernel alone over --batch rows of the size's vocabulary, settings in turn: device time of a draw
        # (settings uploaded, kernel, ids left on the device), draws back to back.
        from llmx_b200.sampling.sampler import sample_async
        raw = dict(QWEN3_8B)
        raw.update(SIZES[args.size])
        vocab = raw["vocab_size"]
        dev_gen = torch.Generator(device="cuda")
        dev_gen.manual_seed(3)
        logits = torch.randn(args.batch, vocab, device="cuda", generator=dev_gen) * 3.0
        settings = {"greedy": SamplingParams(temp=0.0, top_k=0, top_p=1.0),
                    "top_k40_top_p0.95": SamplingParams(temp=0.8, top_k=40, top_p=0.95),
                    "top_k1000": SamplingParams(temp=1.0, top_k=1000, top_p=1.0),
                    "top_p0.95": SamplingParams(temp=1.0, top_k=0, top_p=0.95),
                    "temperature": SamplingParams(temp=1.0, top_k=0, top_p=1.0)}
        line = {"only": "sample", "rows": args.batch, "vocab": vocab, "unit": "us a draw"}
        for name, params in settings.items():
            states = [RequestSampling(params) for _ in range(args.batch)]
            for _ in range(args.warmup):
                sample_async(logits, states).result()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                sample_async(logits, states)
            e1.record()
            torch.cuda.synchronize()
            line[name] = round(e0.elapsed_time(e1) * 1e3 / args.steps, 1)
        print(json.dumps(line))
        return 0
    if args.only == "prefill":
        b = Bench(args.size, args.layers, [], args.context, args.prefill_tokens, args.steps, args.warmup)
        pf_value, pf_ms, pf_sd, pf_frac = b.run_prefill(3, 3)
        line = {"only": "prefill", "value": round(pf_value, 1), "ms": round(pf_ms, 3), "frac": round(pf_frac, 4), "layers": b.layers}
        if args.profile:
            line["profile"] = b.profile_plain_step([StepEntry("profile", b.ids(args.prefill_tokens), [args.prefill_tokens - 1])], f"pp{args.prefill_tokens}")
        print(json.dumps(line))
        return 0
    if args.only == "decode":
        b = Bench(args.size, args.layers, [args.batch], args.context, args.prefill_tokens, args.steps, args.warmup)
        times, launches, _ = b.run_decode(args.batch, args.steps, args.warmup)
        line = {"only": "decode", "value": round(args.batch * 1e3 / times[0], 1), "ms_per_step": round(times[0], 4),
                "batch": args.batch, "context": args.context, "layers": b.layers, "gpu_launches": launches}
        if args.profile:
            rids = [("profile", i) for i in range(args.batch)]
            for rid in rids:
                rc = b.engine.cache.new_request(rid)
                rc.prepare(args.context)
                rc.commit()
            line["profile"] = b.profile_plain_step([StepEntry(rid, [1], [0]) for rid in rids], f"tg{args.batch}")
        print(json.dumps(line))
        return 0
    clocks = ClockSampler()          # clocks and throttle reasons over every timed region below
    clocks.start()
    REPEATS = 3                      # timed regions of K steps each; the headline is the first, mean and sd go beside it
    main_batches = [args.batch] + ([] if args.no_points else [b for b in (1, 64) if b != args.batch])
    try:
        bench = Bench(args.size, args.layers, main_batches, args.context, args.prefill_tokens, args.steps, args.warmup)
    except RuntimeError as e:
        print(f"bench: {e}", file=sys.stderr)
        return 1
    if args.batch not in bench.batches:
        print(f"bench: batch {args.batch} at context {args.context} does not fit; give a smaller --batch, --context or --layers", file=sys.stderr)
        return 1
    for left in bench.left_out:
        print(f"note: the batch {left} point does not fit beside the weights and is left out", file=sys.stderr)
    cfg = bench.cfg
    times, launches, _ = bench.run_decode(args.batch, args.steps, args.warmup, REPEATS)
    ms = times[0]
    value = args.batch * 1e3 / ms
    mean_rate, sd_rate = rate(args.batch, times)
    e2e_value, e2e_ms, h2d = bench.run_generate(args.batch, args.steps, max(args.warmup, 8))
    try:
        native_value, native_ms, native_h2d, native_replays = bench.run_native(args.batch, args.steps, max(args.warmup, 8))
    except Exception as e:          # the point is left out, the line still stands
        print(f"note: the native engine's point is left out: {e}", file=sys.stderr)
        native_value = None
    pf_value, pf_ms, pf_sd, pf_frac = bench.run_prefill(3, 3)
    points = {}
    for b in bench.batches:
        if b == args.batch:
            continue
        t, _, _ = bench.run_decode(b, args.steps if b < 64 else max(args.steps // 2, 8), args.warmup, REPEATS)
        m, sd = rate(b, t)
        points[f"decode_b{b}"] = round(m, 1)
        points[f"decode_b{b}_sd"] = round(sd, 2)
        # the same roofline as the headline's: bytes the step must read over its time, against the copy bandwidth
        points[f"decode_b{b}_hbm_frac"] = round(bench.hbm_frac(b, b * 1e3 / m), 4)
    achieved = bench.decode_bytes(args.batch) / (ms * 1e-3) / 1e9
    model_layers, layers = bench.model_layers, bench.layers
    E, F, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    bench.close()
    # The other published sizes of the architecture (other widths, depths and head counts), each at its own context:
    # the small one is bound by launches and the cache, the large one by 64 GB of weights.
    if not args.no_points and args.size == "8b" and args.layers is None:
        for tag, size, batches, ctx in (("q0_6b", "0.6b", [64], 4096), ("q32b", "32b", [1, 8, 32], 4096)):
            try:
                other = Bench(size, None, batches, ctx, 2048, args.steps, args.warmup)
            except RuntimeError as e:
                print(f"note: {size}: {e}", file=sys.stderr)
                continue
            for b in other.batches:
                t, _, _ = other.run_decode(b, max(args.steps // 2, 8), args.warmup, REPEATS)
                m, sd = rate(b, t)
                points[f"{tag}_decode_b{b}_c{ctx}"] = round(m, 1)
                points[f"{tag}_decode_b{b}_c{ctx}_sd"] = round(sd, 2)
                points[f"{tag}_decode_b{b}_c{ctx}_hbm_frac"] = round(other.hbm_frac(b, b * 1e3 / m), 4)
            v, p_ms, p_sd, frac = other.run_prefill(3, 3)
            points[f"{tag}_prefill_2048"] = round(v, 1)
            points[f"{tag}_prefill_2048_ms_sd"] = round(p_sd, 3)
            points[f"{tag}_prefill_2048_frac"] = round(frac, 4)
            other.close()
    clock_record = clocks.stop()
    ops_tc.check_errors()
    line = {
        "metric": f"decode tok/s at batch {args.batch}, context {args.context} (Qwen3-{args.size.upper()} sizes, bf16, random weights)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "repeats": {"runs": REPEATS, "mean": round(mean_rate, 1), "sd": round(sd_rate, 2)},
        "config": {"model": f"Qwen3-{args.size.upper()} sizes, random weights", "layers": layers, "model_layers": model_layers,
                   "hidden": E, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": F, "vocab": V, "global_batch": args.batch,
                   "seq_len": args.context, "page_size": page, "prefill_tokens": args.prefill_tokens,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (weights and cache read each step)",
                   "history": "synthetic cache contents", "peaks": pk["source"]},
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches,
        "e2e_native": None if native_value is None else {
            "value": round(native_value, 1), "unit": "tok/s", "ms_per_step": round(native_ms, 4), "h2d_bytes_per_step": native_h2d,
            "d2h_bytes_per_step": 4 * args.batch, "replayed_steps": native_replays,
            "what": "the same steps through the native (C++) engine: llmx_engine_add_request / llmx_engine_step"},
        "prefill": {"value": round(pf_value, 1), "tokens": args.prefill_tokens, "ms": round(pf_ms, 3), "ms_sd": round(pf_sd, 3),
                    "frac": round(pf_frac, 4), "peak_tflops": pk["bf16_tflops"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_record,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
