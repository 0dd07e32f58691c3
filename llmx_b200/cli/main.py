"""The command line: `llmx generate MODEL PROMPT_IDS [flags]`, `llmx logits` and `llmx bench`.

Names and meanings of the options are the reference's where it has them
(src/cli/main.cpp:2018-2040 for generate's flags, :544-574 for the execution flags,
:2193-2204 for bench; short forms :119-120; strictness :100-284): exact numeric forms, a flag
given twice is refused, a usage error prints the command's page on stderr and exits with 2.
The tokenizer is outside this engine, so the prompt is token ids: `1,2,3` (commas or spaces),
or `--file F` right after the model for ids in a file.  The reply is printed as ids.
"""
from __future__ import annotations

import sys
import time
from typing import Dict, List, Optional, Tuple

USAGE = """usage:
  llmx generate MODEL (IDS | --file F) [-n N|--max-tokens N] [--temp T] [--topk K] [--topp P] [--min-p P]
                [--penalty P] [--presence-penalty P] [--frequency-penalty P] [--seed S] [--ignore-eos]
                [--dtype auto|bf16|f32] [--ubatch N] [--kv-tokens N] [--cache-type-k T] [--cache-type-v T]
                [--yarn F] [--yarn-original-ctx N] [--device D] [--verbose] [--engine python|native]
      MODEL   a folder with config.json and model.safetensors
      IDS     the prompt as token ids, e.g. 1,2,3
      --yarn F   the rope scaled by YaRN at factor F over the trained length (--yarn-original-ctx N, default the
                 files' declared one, else their context); the model's context becomes F times that length
  llmx logits MODEL (IDS | --file F) [--top K] [--last N] [--per-token] [--dtype auto|bf16|f32] [--ubatch N]
      the K best next tokens (default 5) after each of the last N positions (default 1); --per-token feeds
      the ids one at a time instead of in portions of --ubatch
  llmx bench --model MODEL [--p P] [--n G] [--r R] [--seqs S] [--depth D] [--dtype auto|bf16|f32] [--ubatch N]
             [--profile]
      prompt of P tokens (default 64) and G decoded tokens (default 64), each after a history of D tokens
      (default 0), R repeats (default 3); with --seqs S, S sequences decode together after the prompt each;
      --profile adds the device time of each kernel in one prompt pass and one decode pass
  llmx bench [--size N] [--iters I] [--p P] [--n G]
      without a model: one row through an N x N weight (default 1024), a norm and a per-head norm with rotation
      at width N, I repeats (default 5), then a two-layer model of random weights end to end
"""

SHORT = {"-n": "--max-tokens", "-ctk": "--cache-type-k", "-ctv": "--cache-type-v", "-f": "--file"}


class UsageError(Exception):
    pass


def _int(flag: str, text: str, lo: int, hi: Optional[int] = None) -> int:
    if not text or not (text.isdigit() or (text[0] in "+-" and text[1:].isdigit())) or text[0] == "+":
        raise UsageError(f"{flag}: expected an integer, got '{text}'")
    v = int(text)
    if v < lo or (hi is not None and v > hi):
        raise UsageError(f"{flag}: {v} is out of range")
    return v


def _float(flag: str, text: str, lo: float, hi: float) -> float:
    try:
        v = float(text)
    except ValueError:
        raise UsageError(f"{flag}: expected a number, got '{text}'") from None
    if text.strip() != text or text.lower() in ("nan", "inf", "-inf", "+inf", "infinity") or not (lo <= v <= hi):
        raise UsageError(f"{flag}: {text} is out of range")
    return v


def _ids(text: str) -> List[int]:
    parts = [p for p in text.replace(",", " ").split()]
    if not parts:
        raise UsageError("generate: empty prompt")
    out = []
    for p in parts:
        if not p.isdigit():
            raise UsageError(f"the prompt is token ids, not '{p}'")
        out.append(int(p))
    return out


def _dtype(value: str) -> str:
    table = {"auto": "bfloat16", "bf16": "bfloat16", "f32": "float32"}
    if value not in table:
        raise UsageError("--dtype: expected auto, bf16 or f32 (f16 and int8 are not built in this engine)")
    return table[value]


def _cache_type(given) -> Optional[str]:
    """The cache's element type from --cache-type-k / --cache-type-v (the reference's flags, src/cli/main.cpp:2018-2038),
    or None for the path's own.  Keys and values lie in one storage here, so the two must agree; bf16 and f32 are
    what the kernels take (the reference's f16 default has no kernel in this engine and is refused by name)."""
    k, v = given.get("--cache-type-k"), given.get("--cache-type-v")
    for f, t in (("--cache-type-k", k), ("--cache-type-v", v)):
        if t is not None and t not in ("bf16", "f32"):
            raise UsageError(f"{f} {t}: the cache is bf16 or f32 here (no kernel reads a cache of another type)")
    if k is not None and v is not None and k != v:
        raise UsageError("--cache-type-k and --cache-type-v must agree: keys and values share their pages here")
    t = k if k is not None else v
    return None if t is None else {"bf16": "bfloat16", "f32": "float32"}[t]


def _yarn(given: Dict[str, str]) -> Tuple[Optional[float], Optional[int]]:
    """--yarn F and --yarn-original-ctx N (src/cli/main.cpp:567-571, :597)."""
    yarn = _float("--yarn", given["--yarn"], 1.0, 3.4028234e38) if "--yarn" in given else None
    if yarn == 1.0:
        raise UsageError("--yarn: a factor above 1")
    original = _int("--yarn-original-ctx", given["--yarn-original-ctx"], 1) if "--yarn-original-ctx" in given else None
    if original is not None and yarn is None:
        raise UsageError("--yarn-original-ctx is the length --yarn scales from; give --yarn")
    return yarn, original


def _parse(argv: List[str], valued: Dict[str, str], switches: Tuple[str, ...]):
    """Splits argv into ({flag: text}, [positional]); refuses unknown and repeated flags."""
    given: Dict[str, str] = {}
    positional: List[str] = []
    i = 0
    while i < len(argv):
        a = argv[i]
        f = SHORT.get(a, a)
        if f in valued or f in switches:
            if f in given:
                raise UsageError(f"{a} given twice")
            if f in switches:
                given[f] = "1"
            else:
                if i + 1 >= len(argv):
                    raise UsageError(f"{a} needs a value")
                i += 1
                given[f] = argv[i]
        elif a.startswith("-") and len(a) > 1 and not a[1:].replace(",", "").isdigit():
            raise UsageError(f"unknown flag: {a}")
        else:
            positional.append(a)
        i += 1
    return given, positional


def cmd_generate(argv: List[str]) -> int:
    from ..sampling import SamplingParams
    valued = {k: k for k in ("--max-tokens", "--temp", "--topk", "--topp", "--min-p", "--penalty", "--presence-penalty",
                             "--frequency-penalty", "--seed", "--dtype", "--ubatch", "--kv-tokens", "--cache-type-k",
                             "--cache-type-v", "--device", "--file", "--yarn", "--yarn-original-ctx", "--engine")}
    given, pos = _parse(argv, valued, ("--ignore-eos", "--verbose"))
    if not pos:
        raise UsageError("missing the model")
    model = pos[0]
    if given.get("--engine", "python") not in ("python", "native"):
        raise UsageError("--engine: python or native")
    if "--file" in given:
        if len(pos) > 1:
            raise UsageError(f"a second prompt, '{pos[1]}'")
        with open(given["--file"], "r", encoding="utf-8") as fh:
            prompt = _ids(fh.read())
    else:
        if len(pos) < 2:
            raise UsageError("missing the prompt")
        if len(pos) > 2:
            raise UsageError(f"a second prompt, '{pos[2]}'; quote the prompt to keep its spaces")
        prompt = _ids(pos[1])
    d = SamplingParams()
    fmax = 3.4028234e38
    params = SamplingParams(
        max_tokens=_int("--max-tokens", given.get("--max-tokens", str(d.max_tokens)), 1),
        temp=_float("--temp", given.get("--temp", repr(d.temp)), 0.0, fmax),
        top_k=_int("--topk", given.get("--topk", str(d.top_k)), 0, 2 ** 31 - 1),
        top_p=_float("--topp", given.get("--topp", repr(d.top_p)), 0.0, 1.0),
        min_p=_float("--min-p", given.get("--min-p", repr(d.min_p)), 0.0, 1.0),
        penalty=_float("--penalty", given.get("--penalty", repr(d.penalty)), 1.0, fmax),
        presence_penalty=_float("--presence-penalty", given.get("--presence-penalty", "0"), -2.0, 2.0),
        frequency_penalty=_float("--frequency-penalty", given.get("--frequency-penalty", "0"), -2.0, 2.0),
        seed=_int("--seed", given.get("--seed", "0"), 0, 2 ** 64 - 1),
        ignore_eos="--ignore-eos" in given)
    dtype = _dtype(given.get("--dtype", "auto"))
    kv_dtype = _cache_type(given)
    ubatch = _int("--ubatch", given.get("--ubatch", "2048"), 1)
    kv_tokens = _int("--kv-tokens", given["--kv-tokens"], 1) if "--kv-tokens" in given else None
    if kv_tokens is None:
        kv_tokens = -(-(len(prompt) + params.max_tokens) // 64) * 64
    yarn, yarn_original = _yarn(given)

    if given.get("--engine") == "native":
        return _generate_native(model, prompt, params, dtype, kv_dtype, ubatch, kv_tokens, given, yarn)
    from ..engine.generate import LLM
    t0 = time.perf_counter()
    llm = LLM(model, dtype=dtype, kv_tokens=kv_tokens, ubatch=ubatch, max_seqs=1, device=given.get("--device", "cuda:0"),
              yarn=yarn, yarn_original_ctx=yarn_original, kv_dtype=kv_dtype)
    if "--verbose" in given:
        print(f"load: {time.perf_counter() - t0:.2f} s", file=sys.stderr)
        print(f"prompt tokens: {len(prompt)}")
    out = llm.generate([prompt], params)[0]
    s = llm.stats
    print("ids: " + ",".join(str(t) for t in out.tokens))
    pp_ms, tg_ms = s.prefill_seconds * 1e3, s.decode_seconds * 1e3
    print(f"pp: {len(prompt)} tok, {pp_ms:.0f} ms, {len(prompt) / max(pp_ms / 1e3, 1e-9):.2f} tok/s")
    print(f"tg: {len(out.tokens)} tok, {tg_ms:.0f} ms, {len(out.tokens) / max(tg_ms / 1e3, 1e-9):.2f} tok/s")
    if "--verbose" in given:
        c = llm.engine.cache
        print(f"kv: allocated {c.storage_bytes()} bytes, pages {c.total_pages()}, finish {out.finish_reason}")
    return 0


def _generate_native(model: str, prompt, params, dtype: str, kv_dtype, ubatch: int, kv_tokens: int, given, yarn) -> int:
    """`llmx generate --engine native`: the files read, the request scheduled and the tokens drawn by the native engine
    (csrc/runtime/llmx_engine.h); the same output lines."""
    from ..native_engine import NativeEngine
    if yarn is not None:
        raise UsageError("--yarn: the native loader reads the rope scaling the files declare; use --engine python")
    device = given.get("--device", "cuda:0")
    t0 = time.perf_counter()
    engine = NativeEngine.load(model, dtype=dtype, kv_dtype=kv_dtype, kv_tokens=kv_tokens, ubatch=ubatch, max_requests=1,
                               device=int(device.split(":")[1]) if ":" in device else 0)
    if "--verbose" in given:
        print(f"load: {time.perf_counter() - t0:.2f} s", file=sys.stderr)
        print(f"prompt tokens: {len(prompt)}")
    rid = engine.add_request(prompt, params)
    t0 = time.perf_counter()
    first = None
    while not engine.idle:
        if engine.step() and first is None:
            first = time.perf_counter()
    end = time.perf_counter()
    tokens, reason = engine.output(rid)
    print("ids: " + ",".join(str(t) for t in tokens))
    pp_ms, tg_ms = ((first or end) - t0) * 1e3, (end - (first or end)) * 1e3
    print(f"pp: {len(prompt)} tok, {pp_ms:.0f} ms, {len(prompt) / max(pp_ms / 1e3, 1e-9):.2f} tok/s")
    print(f"tg: {len(tokens)} tok, {tg_ms:.0f} ms, {len(tokens) / max(tg_ms / 1e3, 1e-9):.2f} tok/s")
    if "--verbose" in given:
        print(f"kv: pages {[t for t, _ in engine.pages()]}, steps {engine.steps} ({engine.replays} replayed), finish {reason}")
    engine.close()
    return 0


def cmd_logits(argv: List[str]) -> int:
    """Top logits per position (the reference's `logits`, src/cli/main.cpp:934-980)."""
    import torch
    from ..engine import Engine, EngineOptions, StepEntry
    valued = {k: k for k in ("--top", "--last", "--dtype", "--ubatch", "--device", "--file")}
    given, pos = _parse(argv, valued, ("--per-token",))
    if not pos:
        raise UsageError("missing the model")
    if "--file" in given:
        with open(given["--file"], "r", encoding="utf-8") as fh:
            ids = _ids(fh.read())
        if len(pos) > 1:
            raise UsageError(f"a second text, '{pos[1]}'")
    else:
        if len(pos) != 2:
            raise UsageError("missing the ids" if len(pos) < 2 else f"a second text, '{pos[2]}'")
        ids = _ids(pos[1])
    top = _int("--top", given.get("--top", "5"), 1)
    last = min(_int("--last", given.get("--last", "1"), 1), len(ids))
    ubatch = 1 if "--per-token" in given else _int("--ubatch", given.get("--ubatch", "2048"), 1)
    engine = Engine.from_dir(pos[0], EngineOptions(dtype=_dtype(given.get("--dtype", "auto")),
                                                   kv_tokens=-(-len(ids) // 64) * 64, max_requests=1,
                                                   device=given.get("--device", "cuda:0"), kv_dtype=_cache_type(given)))
    first_wanted = len(ids) - last
    rows = []
    for at in range(0, len(ids), ubatch):
        part = ids[at:at + ubatch]
        want = [i for i in range(len(part)) if at + i >= first_wanted]
        out = engine.step([StepEntry("logits", part, want)])
        if out is not None:
            rows.append(out.float().cpu())
    logits = torch.cat(rows)
    for r, row in enumerate(logits):
        values, tokens = torch.topk(row, min(top, row.numel()))
        best = " ".join(f"{int(t)}:{float(v):.4f}" for v, t in zip(values, tokens))
        print(f"pos {first_wanted + r} after {ids[first_wanted + r]}: {best}")
    return 0


def _bench_ids(seed: int, n: int, vocab: int) -> List[int]:
    """Fixed ids spread over the vocabulary (the reference's bench_ids, src/cli/main.cpp:1185-1189)."""
    state, out = seed & 0xFFFFFFFF, []
    for _ in range(n):
        state = (1664525 * state + 1013904223) & 0xFFFFFFFF
        out.append((state >> 8) % vocab)
    return out


def _timed(fn) -> float:
    import torch
    torch.cuda.synchronize()
    t = time.perf_counter()
    fn()
    torch.cuda.synchronize()
    return time.perf_counter() - t


def _bench_synthetic(size: int, iters: int, p: int, g: int, device: str) -> int:
    """`llmx bench` without a model (src/cli/main.cpp:1097-1167): one row through a square weight, a norm and a
    per-head norm with rotation at width `size`, then a two-layer model with random weights end to end."""
    import torch
    from .. import ops, ops_tc
    from ..engine import Engine, EngineOptions, StepEntry
    from ..engine.decode_loop import DecodeSession
    from ..registry import architecture_of
    dev = torch.device(device)
    with torch.cuda.device(dev):
        x = torch.full((1, size), 0.5, device=dev)
        w = (torch.randn(size, size, device=dev) * 0.02).to(torch.bfloat16)
        out = torch.zeros(1, size, device=dev)
        xb = x.to(torch.bfloat16)
        if size % 8 == 0:
            product = lambda: ops_tc.gemm_tc(xb, w, out)
        else:                                   # the tensor-core product wants rows of 16 bytes
            product = lambda: ops.gemm_plain(xb, w, out, False)
        src = torch.sin(torch.arange(size, device=dev, dtype=torch.float32) * 0.01).reshape(1, size)
        weight = torch.full((size,), 0.1, device=dev)
        dst = torch.empty(1, size, device=dev)
        half = size // 2
        cos = torch.full((1, half), 0.99500417, device=dev)
        sin = torch.full((1, half), 0.09983342, device=dev)
        zero = torch.zeros(1, dtype=torch.int32, device=dev)
        cache = torch.zeros(1, 2, 1, 16, size, device=dev)
        q_out = torch.empty(1, size, device=dev)
        qkv = torch.cat([src, src, src], dim=1).contiguous()
        rope = lambda: ops.head_norm_rope_kv(qkv, 1, 1, size, weight, weight, 1e-6, cos, sin, zero, zero, q_out, cache)
        results = []
        for fn in (product, lambda: ops.rmsnorm(src, weight, 1e-6, dst), rope):
            fn()
            results.append(_timed(lambda: [fn() for _ in range(iters)]) / iters * 1e3)
        mm_ms, rn_ms, rp_ms = results
        print("bench: matmul %dx%d  %8.3f ms  %8.2f GFLOPS" % (size, size, mm_ms, 2.0 * size * size / (mm_ms * 1e6)))
        print("bench: rms_norm n=%d  %8.3f ms" % (size, rn_ms))
        print("bench: norm_rope n=%d  %8.3f ms" % (size, rp_ms))
        # End to end on a small model of random weights: 2 layers, width 256 (src/cli/main.cpp:1150-1165).
        # (a config.json's worth of keys, read through the registry like any model's)
        raw = dict(model_type="qwen3", num_hidden_layers=2, hidden_size=256, intermediate_size=1024, num_attention_heads=8,
                   num_key_value_heads=2, head_dim=32, vocab_size=512, max_position_embeddings=max(2048, p + g + 64))
        cfg = architecture_of(raw).config_cls.from_dict(raw)
        engine = Engine.from_config(cfg, 12345, EngineOptions(kv_tokens=-(-(p + g + 64) // 64) * 64, max_requests=1,
                                                              device=device))
        prompt, gen = _bench_ids(12345, p, 512), _bench_ids(777, g, 512)
        engine.step([StepEntry("w", prompt, [p - 1])])                    # untimed: loads the kernels
        engine.end("w")
        pre = _timed(lambda: engine.step([StepEntry("s", prompt, [p - 1])]))
        session = DecodeSession(engine, ["s"], use_graph=False)
        dec = _timed(lambda: [session.step([t]) for t in gen])
        engine.end("s")
        print("bench: prefill %3d tok  %8.3f ms  %8.1f tok/s" % (p, pre * 1e3, p / pre))
        print("bench: decode  %3d tok  %8.3f ms  %8.1f tok/s" % (g, dec * 1e3, g / dec))
    ops_tc.check_errors()
    return 0


def cmd_bench(argv: List[str]) -> int:
    """`llmx bench` (src/cli/main.cpp:1192-1320, :2181-2222): with --model, prompt and decode rates of the model as
    mean +- sd over R runs after one untimed warm-up, fixed ids, sampling outside the timer; the prompt
    test and a single sequence's decode test run after a history of --depth tokens, --seqs S sequences decode
    together after the prompt each.
    Without --model, the kernels at width --size and a two-layer random model."""
    import torch
    from ..engine import Engine, EngineOptions, StepEntry
    valued = {k: k for k in ("--model", "--p", "--n", "--r", "--seqs", "--depth", "--dtype", "--device", "--ubatch",
                             "--size", "--iters")}
    given, pos = _parse(argv, valued, ("--profile",))
    if pos:
        raise UsageError(f"bench takes flags only, not '{pos[0]}'")
    p = _int("--p", given.get("--p", "64"), 1)
    g = _int("--n", given.get("--n", "64"), 1)
    model_only = next((f for f in ("--r", "--seqs", "--depth", "--profile", "--dtype", "--ubatch") if f in given), None)
    synthetic_only = next((f for f in ("--size", "--iters") if f in given), None)
    if "--model" not in given:
        if model_only:
            raise UsageError(f"{model_only} takes --model")
        return _bench_synthetic(_int("--size", given.get("--size", "1024"), 32), _int("--iters", given.get("--iters", "5"), 1),
                                p, g, given.get("--device", "cuda:0"))
    if synthetic_only:
        raise UsageError(f"{synthetic_only} is for the synthetic bench, not --model")
    reps = _int("--r", given.get("--r", "3"), 1)
    seqs = _int("--seqs", given.get("--seqs", "1"), 1)
    depth = _int("--depth", given.get("--depth", "0"), 0)
    ubatch = _int("--ubatch", given.get("--ubatch", "2048"), 1)
    dtype = _dtype(given.get("--dtype", "auto"))
    reach = max(p + g, depth + p) if seqs > 1 else depth + max(p, g)
    kv = (-(-(reach + 2) // 64) * 64 + 64) * seqs
    engine = Engine.from_dir(given["--model"], EngineOptions(dtype=dtype, kv_tokens=kv, max_requests=seqs,
                                                             device=given.get("--device", "cuda:0"), record_after=2,
                                                             kv_dtype=_cache_type(given)))
    if reach > engine.max_positions:
        raise UsageError(f"the tests reach {reach} tokens, past the model's context of {engine.max_positions}")
    vocab = engine.model.vocab_size
    prompt, gen, history = _bench_ids(12345, p, vocab), _bench_ids(777, g, vocab), _bench_ids(4242, depth, vocab)

    from ..engine.decode_loop import DecodeSession

    def feed(rid, ids, want_last, record=True):
        for at in range(0, len(ids), ubatch):
            part = ids[at:at + ubatch]
            last = at + ubatch >= len(ids)
            engine.step([StepEntry(rid, part, [len(part) - 1] if want_last and last else [])], record=record)

    def pp(record=True) -> float:
        if depth:
            feed("s", history, False)
        dt = _timed(lambda: feed("s", prompt, True, record))
        engine.end("s")
        return p / dt

    def tg(profile=None) -> float:
        ids = list(range(seqs)) if seqs > 1 else ["s"]
        for rid in ids:
            feed(rid, prompt if seqs > 1 else (history or [gen[0]]), False)
        session = DecodeSession(engine, ids, use_graph=profile is None)
        for _ in range(2):                            # the session's plain step and its recording are not timed
            session.step([gen[0]] * seqs)
        if profile is not None:
            with profile:
                session.step([gen[0]] * seqs)

        def decode():
            for t in gen:
                session.step([t] * seqs)               # a server reads each pass's logits; here they stay on the device
        dt = _timed(decode)
        session.close()
        for rid in ids:
            engine.end(rid)
        return g * seqs / dt

    tg()                                               # untimed: loads the kernels
    for _ in range(4):                                 # untimed: a shape that keeps coming gets recorded
        pp()
    ppv = [pp() for _ in range(reps)]
    tgv = [tg() for _ in range(reps)]

    def report(what: str, n: int, v: List[float]) -> None:
        m = sum(v) / len(v)
        sd = (sum((x - m) ** 2 for x in v) / (len(v) - 1)) ** 0.5 if len(v) > 1 else 0.0
        at = f" @ d{depth}" if depth else ""
        print("bench: %s%d%s  %8.2f +- %.2f tok/s  (%d runs)" % (what, n, at, m, sd, len(v)))
    report("pp", p, ppv)
    report(f"x{seqs} tg" if seqs > 1 else "tg", g, tgv)
    if "--profile" in given:
        # One prompt pass and one decode pass as plain steps (a replayed recording makes no calls to time).
        from .. import ops
        if depth:
            feed("s", history, False)
        with ops.kernel_times() as times:
            feed("s", prompt, True, record=False)
        engine.end("s")
        print("\n".join(times.lines(f"pp{p}")))
        times = ops.kernel_times()
        tg(profile=times)
        print("\n".join(times.lines(f"x{seqs} tg" if seqs > 1 else "tg")))
    from .. import ops_tc
    ops_tc.check_errors()
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        if not argv or argv[0] in ("-h", "--help", "help"):
            print(USAGE)
            return 0
        cmd, rest = argv[0], argv[1:]
        if cmd == "generate":
            return cmd_generate(rest)
        if cmd == "bench":
            return cmd_bench(rest)
        if cmd == "logits":
            return cmd_logits(rest)
        raise UsageError(f"unknown command: {cmd}")
    except UsageError as e:
        print(f"llmx: {e}\n{USAGE}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
