"""The engine against the plain implementation, under every way of cutting and batching.

Each test replays the same requests through `Engine.step` in a different way and compares every
position's logits with `tests/plain_qwen3.py` (whole sequences, no cache).  float32 is held to
1e-4 of the logit scale; bfloat16 is compared with the plain implementation rounding what the
bfloat16 path rounds (inputs of products, cache) and held to the configuration's frozen budget (tests/configs.py:
twice the error measured for it), as a fraction of the logit scale.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers
from configs import BF16_BUDGET, BF16_UNCALIBRATED, CONFIGS

pytestmark = pytest.mark.gpu

def tol(dtype, name=None):
    """The most a logit may differ from the plain implementation, as a fraction of the logit scale: 1e-4 in float32;
    in bfloat16 the configuration's frozen budget (tests/configs.py)."""
    return 1e-4 if dtype == "float32" else BF16_BUDGET.get(name, BF16_UNCALIBRATED)


LENGTHS = [70, 1, 9, 40, 133, 33, 5, 96]


def _requests(name):
    vocab = CONFIGS[name][0]["vocab_size"]
    return {f"r{i}": helpers.random_ids(vocab, n, seed=100 * i + n) for i, n in enumerate(LENGTHS)}


def _engine(model_dirs, name, dtype, kv_tokens):
    from llmx_b200.engine import Engine, EngineOptions
    d16, d32, page = model_dirs[name]
    folder = d32 if dtype == "float32" else d16
    return folder, Engine.from_dir(folder, EngineOptions(dtype=dtype, kv_tokens=kv_tokens, page_size=page,
                                                         max_requests=8))


def _check(engine, folder, steps, requests, dtype, name=None):
    from llmx_b200 import ops_tc
    got = helpers.run_trace(engine, steps)
    ops_tc.check_errors()
    engine.cache.check()
    assert engine.cache.used_pages() == [0] * len(engine.cache.groups)
    wanted = sum(len(e["want"]) for s in steps for e in s["entries"])
    assert len(got) == wanted == sum(len(v) for v in requests.values())
    worst, scale, where = helpers.compare(got, requests, folder, dtype == "bfloat16")
    assert worst <= tol(dtype, name) * scale, f"largest difference {worst:.3e} at {where} (logit scale {scale:.3f})"
    return worst, scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
class TestCuttings:
    def test_whole(self, model_dirs, name, dtype):
        requests = _requests(name)
        steps = helpers.trace_whole(requests)
        folder, engine = _engine(model_dirs, name, dtype, helpers.tokens_needed(steps))
        _check(engine, folder, steps, requests, dtype, name)

    def test_last_32_one_by_one(self, model_dirs, name, dtype):
        requests = _requests(name)
        steps = helpers.trace_tail_decoded(requests, 32)
        folder, engine = _engine(model_dirs, name, dtype, helpers.tokens_needed(steps))
        _check(engine, folder, steps, requests, dtype, name)

    def test_portions_of_changing_size(self, model_dirs, name, dtype):
        requests = _requests(name)
        steps = helpers.trace_portions(requests)
        assert min(len(e["tokens"]) for s in steps for e in s["entries"] if len(e["tokens"]) > 1) == 2
        folder, engine = _engine(model_dirs, name, dtype, helpers.tokens_needed(steps))
        _check(engine, folder, steps, requests, dtype, name)

    def test_mixed_with_pages_used_again(self, model_dirs, name, dtype):
        requests = _requests(name)
        steps = helpers.trace_mixed(requests)
        assert max(len(s["entries"]) for s in steps) == 4
        need = helpers.tokens_needed(steps)
        assert need < sum(-(-len(v) // 64) * 64 for v in requests.values())   # the pool cannot hold them all at once
        folder, engine = _engine(model_dirs, name, dtype, need)
        seen = set()
        reused = False
        from llmx_b200.engine import StepEntry
        # Watch the block tables as the trace runs: a page id must come back after it was given up.
        got = {}
        at = {}
        for s in steps:
            logits = engine.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
            rows = logits.float().cpu().numpy()
            k = 0
            for e in s["entries"]:
                base = at.get(e["id"], 0)
                for w in e["want"]:
                    got[(e["id"], base + w)] = rows[k]
                    k += 1
                at[e["id"]] = base + len(e["tokens"])
            held = {p for rc in engine.cache.live.values() for p in rc.tables[0].pages}
            for rid in s["end"]:
                gone = set(engine.cache.live[rid].tables[0].pages)
                engine.end(rid)
                seen |= gone
                held -= gone
            reused = reused or bool(seen & held)
            engine.cache.check()
        assert reused, "no page was used again; the pool was not tight enough to test reuse"
        worst, scale, where = helpers.compare(got, requests, folder, dtype == "bfloat16")
        assert worst <= tol(dtype, name) * scale, f"largest difference {worst:.3e} at {where} (logit scale {scale:.3f})"


@pytest.mark.parametrize("name", ["B", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_dirs, name, dtype):
    """A short prompt, then 300 tokens one by one across many pages."""
    vocab = CONFIGS[name][0]["vocab_size"]
    requests = {"long": helpers.random_ids(vocab, 320, seed=7)}
    steps = helpers.trace_tail_decoded(requests, tail=300)
    folder, engine = _engine(model_dirs, name, dtype, 320)
    _check(engine, folder, steps, requests, dtype, name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_first_tokens_of_a_sequence(model_dirs, name, dtype):
    """Positions 0, 1, 2: a single key, the first page's first slots, decoded one by one from nothing."""
    vocab = CONFIGS[name][0]["vocab_size"]
    requests = {"s": helpers.random_ids(vocab, 3, seed=3), "t": helpers.random_ids(vocab, 1, seed=4)}
    steps = helpers.trace_tail_decoded(requests, tail=3)
    folder, engine = _engine(model_dirs, name, dtype, 128)
    _check(engine, folder, steps, requests, dtype, name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["python", "native"])
def test_trace_run_program(model_dirs, tmp_path, dtype, which):
    """bin/trace_run as a user runs it: JSON steps on standard input, .f32 files out, `done` lines; through the Python
    engine (the default) and through the native one."""
    name = "B"
    d16, d32, page = model_dirs[name]
    folder = d32 if dtype == "float32" else d16
    vocab = CONFIGS[name][0]["vocab_size"]
    requests = {f"q{i}": helpers.random_ids(vocab, n, seed=50 + i) for i, n in enumerate([45, 3, 80, 20, 64])}
    steps = helpers.trace_mixed(requests, tail=5)
    need = helpers.tokens_needed(steps)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(need)] + (["--engine", "native"] if which == "native" else []),
                          input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    got = helpers.read_trace_output(steps, str(out), vocab)
    worst, scale, where = helpers.compare(got, requests, folder, dtype == "bfloat16")
    assert worst <= tol(dtype, name) * scale, f"largest difference {worst:.3e} at {where} (logit scale {scale:.3f})"


def test_step_refusals(model_dirs):
    from llmx_b200.cache import CacheExhausted
    from llmx_b200.engine import StepEntry, StepError
    folder, engine = _engine(model_dirs, "A", "float32", 64)
    with pytest.raises(StepError):
        engine.step([])
    with pytest.raises(StepError):
        engine.step([StepEntry("a", [], [])])
    with pytest.raises(StepError):
        engine.step([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])
    with pytest.raises(StepError):
        engine.step([StepEntry("a", [256], [0])])
    with pytest.raises(StepError):
        engine.step([StepEntry("a", [1, 2], [2])])
    # Pages run out: nothing is kept, and the same request fits once room is made.
    engine.step([StepEntry("a", list(range(48)), [47])])
    with pytest.raises(CacheExhausted):
        engine.step([StepEntry("b", list(range(40)), [0])])
    engine.cache.check()
    assert "b" not in engine.cache.live and engine.length("a") == 48
    engine.end("a")
    assert engine.step([StepEntry("b", list(range(40)), [0])]).shape == (1, 256)
    engine.end("b")
    assert engine.cache.used_pages() == [0]


def _sharpened(model_dirs, tmp_path_factory, names, factor):
    import torch
    from llmx_b200.weights import TensorDirectory, write_safetensors
    out = {}
    for name in names:
        made = []
        for src in model_dirs[name][:2]:
            d = str(tmp_path_factory.mktemp(f"sharp_{name}"))
            t = TensorDirectory(src)
            tensors = {}
            for n in t.names():
                x = t.tensor(n).clone()
                if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
                    x = x * factor
                tensors[n] = x
            write_safetensors(os.path.join(d, "model.safetensors"), tensors)
            with open(os.path.join(src, "config.json")) as f, open(os.path.join(d, "config.json"), "w") as g:
                g.write(f.read())
            made.append(d)
        out[name] = (made[0], made[1], model_dirs[name][2])
    return out


@pytest.fixture(scope="module")
def sharp_model_dirs(model_dirs, tmp_path_factory):
    """Models whose attention is sharp: the q/k norm weights are scaled by 4, so scores spread over +-16 and a
    row's output hangs on a few keys anywhere in its history.  With the random weights' nearly uniform attention
    a key that is dropped or read from the wrong page changes a row by ~1/length; here it changes it outright."""
    return _sharpened(model_dirs, tmp_path_factory, ("B", "D"), 4.0)


@pytest.fixture(scope="module")
def half_sharp_model_dirs(model_dirs, tmp_path_factory):
    """The same with the weights doubled (scores four times as wide as the random model's): sharp enough that a key
    read from the wrong place moves a logit far beyond the budget, mild enough that one bfloat16 step in a query or
    key does not."""
    return _sharpened(model_dirs, tmp_path_factory, ("B", "D", "E"), 2.0)


@pytest.mark.parametrize("name", ["B", "D", "E"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_sharpened_attention_in_bfloat16_under_cutting(half_sharp_model_dirs, name, cutting):
    """The bfloat16 path's own choices inside the engine -- the product that finishes its heads, the decode kernel
    that makes its own queries and keys, the tiled prefill kernels, recorded steps -- with attention that hangs on
    single keys: every logit within the sharpened model's frozen budget of the plain implementation."""
    vocab = CONFIGS[name][0]["vocab_size"]
    requests = {f"s{i}": helpers.random_ids(vocab, n, seed=300 + i) for i, n in enumerate([200, 37, 150, 9, 64])}
    make = {"whole": helpers.trace_whole, "tail": helpers.trace_tail_decoded, "portions": helpers.trace_portions,
            "mixed": helpers.trace_mixed}[cutting]
    steps = make(requests)
    folder, engine = _engine(half_sharp_model_dirs, name, "bfloat16", helpers.tokens_needed(steps))
    _check(engine, folder, steps, requests, "bfloat16", "sharp:" + name)


@pytest.mark.parametrize("name", ["B", "D"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_sharp_attention_under_cutting(sharp_model_dirs, name, cutting):
    """The float32 path against the plain implementation with attention that hangs on single far keys.

    Only float32: with scores of +-16 one bfloat16 step in q or k moves a softmax weight by several per cent, so in
    bfloat16 the comparison would measure that rounding, not the cache (two bfloat16 runs of the same prompt cut
    differently differ by 4 % of the logit scale here, from the order of float sums alone).  The bfloat16 kernels
    meet keys that stand out in tests/test_kernels_gpu.py (spike=True), on inputs that are bfloat16 to begin with."""
    vocab = CONFIGS[name][0]["vocab_size"]
    requests = {f"s{i}": helpers.random_ids(vocab, n, seed=300 + i) for i, n in enumerate([200, 37, 150, 9, 64])}
    make = {"whole": helpers.trace_whole, "tail": helpers.trace_tail_decoded, "portions": helpers.trace_portions,
            "mixed": helpers.trace_mixed}[cutting]
    steps = make(requests)
    folder, engine = _engine(sharp_model_dirs, name, "float32", helpers.tokens_needed(steps))
    _check(engine, folder, steps, requests, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_yarn_forced_by_the_options(model_dirs, tmp_path, dtype):
    """`EngineOptions.yarn` (the command line's --yarn) scales the rope of a model whose files declare none and
    stretches its context: the same weights under a config.json that declares that scaling give the plain
    implementation's logits, on a prompt longer than the files' own context."""
    import json
    import shutil
    from llmx_b200.engine import Engine, EngineOptions
    d16, d32, page = model_dirs["A"]
    folder = d32 if dtype == "float32" else d16
    declared = dict(CONFIGS["A"][0], max_position_embeddings=1024,
                    rope_scaling=dict(rope_type="yarn", factor=4.0, original_max_position_embeddings=256))
    twin = tmp_path / "declared"
    twin.mkdir()
    shutil.copy(f"{folder}/model.safetensors", twin / "model.safetensors")
    (twin / "config.json").write_text(json.dumps(declared))
    requests = {"y": helpers.random_ids(CONFIGS["A"][0]["vocab_size"], 600, seed=5)}      # past the files' 512
    steps = helpers.trace_portions(requests, portions=(300, 2, 170, 128))
    engine = Engine.from_dir(folder, EngineOptions(dtype=dtype, kv_tokens=helpers.tokens_needed(steps), page_size=page,
                                                   max_requests=2, yarn=4.0, yarn_original_ctx=256))
    assert engine.max_positions == 1024
    _check(engine, str(twin), steps, requests, dtype)


def test_kernel_times_of_a_plain_step(model_dirs):
    """`ops.kernel_times`: device time by exported kernel function over the calls of a plain step (what
    `llmx bench --profile` prints); the step's result is what it is without the timing."""
    import torch
    from llmx_b200 import ops
    from llmx_b200.engine import StepEntry
    folder, engine = _engine(model_dirs, "B", "bfloat16", 256)
    ids = helpers.random_ids(CONFIGS["B"][0]["vocab_size"], 40, seed=3)
    plain = engine.step([StepEntry("a", ids, [39])]).clone()
    engine.end("a")
    with ops.kernel_times() as times:
        timed = engine.step([StepEntry("a", ids, [39])]).clone()
    engine.end("a")
    assert torch.equal(plain, timed)
    layers = CONFIGS["B"][0]["num_hidden_layers"]
    assert times.calls >= 6 * layers and times.total_ms > 0 and times.idle_ms >= 0
    assert times.by_function["llmx_rmsnorm"][0] == 2 * layers + 1
    assert sum(n for n, _ in times.by_function.values()) == times.calls
    report = times.lines("pp40")
    assert report[0].startswith("profile pp40:") and report[-1].startswith("profile pp40: idle")
    with pytest.raises(ops.KernelError):
        with ops.kernel_times():
            with ops.kernel_times():
                pass
    assert ops._timed_calls is None


WIDE = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=4096, intermediate_size=12288, num_attention_heads=32, num_key_value_heads=8,
    head_dim=128, vocab_size=32003, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
    max_position_embeddings=4096)


@pytest.fixture(scope="module")
def wide_model_dir(tmp_path_factory):
    """Two layers with the widths of Qwen3-8B (and a vocabulary that is no multiple of anything), so that the
    kernels run at the sizes they are built for: full tensor-core tiles, 64 k blocks, 32 heads over 8 kv heads."""
    import torch
    from llmx_b200.config import Qwen3Config
    from llmx_b200.weights import write_random_model
    d = str(tmp_path_factory.mktemp("wide"))
    write_random_model(d, Qwen3Config.from_dict(WIDE), seed=9, dtype=torch.bfloat16)
    return d


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_of_8b_width_under_cutting(wide_model_dir, dtype):
    """The stored weights are bfloat16, exact in both paths; the float32 path widens them."""
    from llmx_b200.engine import Engine, EngineOptions
    requests = {f"w{i}": helpers.random_ids(WIDE["vocab_size"], n, seed=40 + i) for i, n in enumerate([150, 70, 33, 2])}
    for make in (helpers.trace_whole, helpers.trace_tail_decoded, helpers.trace_portions, helpers.trace_mixed):
        steps = make(requests)
        engine = Engine.from_dir(wide_model_dir, EngineOptions(dtype=dtype, kv_tokens=helpers.tokens_needed(steps),
                                                               page_size=16, max_requests=4))
        _check(engine, wide_model_dir, steps, requests, dtype, "wide")
        del engine


def test_long_prompts_at_8b_width(wide_model_dir):
    """Steps of 256 rows and more let the q/k/v product norm, rotate and store its heads itself (one head or two a tile); shorter steps go through the float32 output and the per-head kernel.  Long prompts whole, in
    portions on both sides of those sizes, and two prompts in one step: every logit against the plain
    implementation, so keys stored by either way serve rows computed by the other."""
    from llmx_b200 import ops_tc
    from llmx_b200.engine import Engine, EngineOptions
    vocab = WIDE["vocab_size"]
    requests = {"L": helpers.random_ids(vocab, 1100, seed=61), "M": helpers.random_ids(vocab, 300, seed=62)}
    together = [{"step": 0, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}
                                        for rid, ids in requests.items()], "end": list(requests)}]
    traces = [helpers.trace_whole(requests), helpers.trace_portions(requests, portions=(520, 7, 260, 64, 249, 300)),
              together]
    assert {ops_tc.heads_tile(n, 32, 8) for n in (1100, 520, 300, 260)} == {128, 256}
    assert ops_tc.heads_tile(249, 32, 8) == 0
    for steps in traces:
        engine = Engine.from_dir(wide_model_dir, EngineOptions(dtype="bfloat16", kv_tokens=helpers.tokens_needed(steps),
                                                               page_size=16, max_requests=4))
        _check(engine, wide_model_dir, steps, requests, "bfloat16", "wide")
        del engine


def test_long_portions_recorded_at_8b_width(wide_model_dir):
    """The same shapes of long steps come again and are replayed from recordings: the q/k/v product that finishes its
    heads and the prefill attention's key ranges (chosen when the step is recorded) inside a recording, on other
    pages from the second time on, against the plain implementation."""
    from llmx_b200 import ops_tc
    from llmx_b200.engine import Engine, EngineOptions
    vocab = WIDE["vocab_size"]
    engine = Engine.from_dir(wide_model_dir, EngineOptions(dtype="bfloat16", kv_tokens=4096, page_size=16, max_requests=4,
                                                           record_after=1))
    from llmx_b200 import ops_attn
    assert ops_attn.prefill_shape(1, 8, 4, 280, 2200, 0)[1] > 1                # 280 rows after 1,920 keys: key ranges
    requests = {"x": helpers.random_ids(vocab, 2200, seed=70)}
    steps = helpers.trace_portions(requests, portions=(1920, 280))
    for run in range(3):
        if run == 1:
            engine.step([helpers_entry("pad", helpers.random_ids(vocab, 50, seed=1))])      # other pages from here on
        got = helpers.run_trace(engine, steps, record=True)
        ops_tc.check_errors()
        worst, scale, where = helpers.compare(got, requests, wide_model_dir, True)
        assert worst <= tol("bfloat16", "wide") * scale, f"run {run}: largest difference {worst:.3e} at {where}"
    assert len(engine.step_recordings) == 2
    engine.end("pad")
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "wide"])
def test_recorded_steps_of_any_shape(model_dirs, wide_model_dir, name, dtype):
    """A step's shape that comes again is recorded and replayed (prompt portions, portions beside decoding rows,
    several rows of one request): the same trace run four times over, the last runs from recordings, each against
    the plain implementation; the pool is so small that later runs find their pages elsewhere."""
    from llmx_b200 import ops_tc
    from llmx_b200.engine import Engine, EngineOptions
    if name == "wide":
        folder, page, vocab = wide_model_dir, 16, WIDE["vocab_size"]
        lengths = [150, 70, 33, 2]
    else:
        d16, d32, page = model_dirs[name]
        folder, vocab = (d32 if dtype == "float32" else d16), CONFIGS[name][0]["vocab_size"]
        lengths = [70, 9, 40, 33]
    requests = {f"q{i}": helpers.random_ids(vocab, n, seed=7 + i) for i, n in enumerate(lengths)}
    steps = helpers.trace_mixed(requests)
    engine = Engine.from_dir(folder, EngineOptions(dtype=dtype, kv_tokens=helpers.tokens_needed(steps) + 3 * page,
                                                   page_size=page, max_requests=5, record_after=2))
    for run in range(4):
        if run == 2:                                   # shift the pool: the recorded steps must not remember pages
            engine.step([helpers_entry("pad", helpers.random_ids(vocab, 2 * page + 1, seed=1))])
        got = helpers.run_trace(engine, steps, record=True)
        ops_tc.check_errors()
        worst, scale, where = helpers.compare(got, requests, folder, dtype == "bfloat16")
        assert worst <= tol(dtype, name) * scale, f"run {run}: largest difference {worst:.3e} at {where} (logit scale {scale:.3f})"
    assert len(engine.step_recordings) > 0
    replayed = sum(1 for s in steps if (tuple(len(e["tokens"]) for e in s["entries"])) in {k[0] for k in engine.step_recordings})
    assert replayed >= len(steps) // 2
    engine.end("pad")
    engine.cache.check()
    assert engine.cache.used_pages() == [0] * len(engine.cache.groups)


def helpers_entry(rid, tokens):
    from llmx_b200.engine import StepEntry
    return StepEntry(rid, tokens, [])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "wide"])
def test_decode_sessions_replay_their_recordings(model_dirs, wide_model_dir, name, dtype):
    """Prompts by plain steps, then their last tokens one by one through decode sessions: the first step of a new
    batch size is plain, the next records, the rest replay; token ids come from the host or from a device tensor;
    a request leaves and the remaining ones carry on in a new session; every row against the plain implementation."""
    import torch
    from llmx_b200 import ops_tc
    from llmx_b200.engine import Engine, EngineOptions, StepEntry
    from llmx_b200.engine.decode_loop import DecodeSession
    if name == "wide":
        folder, page, vocab = wide_model_dir, 16, WIDE["vocab_size"]
    else:
        d16, d32, page = model_dirs[name]
        folder, vocab = (d32 if dtype == "float32" else d16), CONFIGS[name][0]["vocab_size"]
    lengths = {"a": 70, "b": 41, "c": 55}
    requests = {rid: helpers.random_ids(vocab, n, seed=90 + n) for rid, n in lengths.items()}
    tail = 24
    engine = Engine.from_dir(folder, EngineOptions(dtype=dtype, kv_tokens=4 * 96, page_size=page, max_requests=4))
    got = {}
    for rid, ids in requests.items():
        head = len(ids) - tail
        logits = engine.step([StepEntry(rid, ids[:head], list(range(head)))]).float().cpu().numpy()
        for p in range(head):
            got[(rid, p)] = logits[p]
    live = list(requests)
    at = {rid: len(requests[rid]) - tail for rid in live}
    session = DecodeSession(engine, live)
    for step in range(tail):
        if step == 10:                      # "b" leaves: the others carry on in a session (and a recording) of two
            session.close()
            engine.end("b")
            live.remove("b")
            session = DecodeSession(engine, live)
        tokens = [requests[rid][at[rid]] for rid in live]
        feed = torch.tensor(tokens, dtype=torch.int32, device="cuda") if step % 3 == 2 else tokens
        logits = session.step(feed).float().cpu().numpy()
        for k, rid in enumerate(live):
            got[(rid, at[rid])] = logits[k]
            at[rid] += 1
    session.close()
    ops_tc.check_errors()
    assert {b for (b, _room) in engine.decode_recordings} == {3, 2}
    requests_seen = {rid: requests[rid][:at[rid]] for rid in requests}
    worst, scale, where = helpers.compare({k: v for k, v in got.items() if k[1] < len(requests_seen[k[0]])}, requests_seen,
                                          folder, dtype == "bfloat16")
    assert worst <= tol(dtype, name) * scale, f"largest difference {worst:.3e} at {where} (logit scale {scale:.3f})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_hugging_face_golden_of_odd_sizes(tmp_path, dtype):
    """The engine at width 37, head width 42, vocabulary 257 (sizes that are multiples of nothing), tied and untied,
    against logits Hugging Face's Qwen3 gave (tests/hf_anchor.py): float32 within the reference's own bound for this
    comparison, whole and with the last tokens decoded one by one; bfloat16 against the plain implementation."""
    import json
    import torch
    import hf_anchor
    from llmx_b200.engine import Engine, EngineOptions, StepEntry
    from llmx_b200.weights import write_safetensors
    fixtures = hf_anchor.fixtures()
    if fixtures is None:
        pytest.skip("the golden file is not at hand")
    for tied, cfg, w, cases in fixtures:
        folder = tmp_path / f"hf_{tied}_{dtype}"
        folder.mkdir()
        store = torch.float32 if dtype == "float32" else torch.bfloat16
        write_safetensors(str(folder / "model.safetensors"), {n: torch.from_numpy(a).to(store) for n, a in w.items()})
        (folder / "config.json").write_text(json.dumps(cfg))
        engine = Engine.from_dir(str(folder), EngineOptions(dtype=dtype, kv_tokens=64, page_size=4, max_requests=2))
        for ids, want in cases:
            whole = engine.step([StepEntry("w", ids, [len(ids) - 1])]).float().cpu().numpy()[0]
            engine.end("w")
            for t in ids:
                last = engine.step([StepEntry("d", [t], [0])]).float().cpu().numpy()[0]
            engine.end("d")
            if dtype == "float32":
                assert np.abs(whole - want).max() <= hf_anchor.BOUND and np.abs(last - want).max() <= hf_anchor.BOUND
            else:
                ref = helpers.reference_logits(str(folder), ids, True)[-1]
                scale = float(np.abs(ref).max())
                assert np.abs(whole - ref).max() <= tol(dtype) * scale and np.abs(last - ref).max() <= tol(dtype) * scale
        engine.cache.check()


# ---------------------------------------------------------------------------------------------
# What a failed step leaves behind, rolling back, cache types, invariance, memory.
def _products(dtype):
    return "llmx_gemm_plain" if dtype == "float32" else "llmx_gemm_tc"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_that_fails_inside_the_forward_pass_leaves_every_request_where_it_was(model_dirs, dtype):
    """The reference's tests fail an operation of their backend in mid-pass, after keys were written, and check that
    every length is back and the same prompt again is exact (tests/tiny_qwen.hpp:104-148).  Here the failure is made
    on the host: the sixth matrix product of the step (the second layer's output projection: both layers' keys of
    the portion are in their pages by then) returns an error instead of launching.  First in a step that holds a
    portion of a live request beside a new request, then in a plain decode step, then in a replayed one."""
    import torch
    from llmx_b200 import ops_tc, runtime
    from llmx_b200.engine import StepEntry
    from llmx_b200.engine.decode_loop import DecodeSession
    vocab = CONFIGS["D"][0]["vocab_size"]
    a_ids, b_ids = helpers.random_ids(vocab, 60, seed=1), helpers.random_ids(vocab, 22, seed=2)
    folder, engine = _engine(model_dirs, "D", dtype, 256)
    _, clean = _engine(model_dirs, "D", dtype, 256)
    loose = 0.0 if dtype == "float32" else 2e-3        # bfloat16 sums pieces with atomics: the last bits move from run to run

    def same(x, y):
        if loose == 0.0:
            return torch.equal(x, y)
        return float((x - y).abs().max()) <= loose * float(y.abs().max())

    first = [StepEntry("a", a_ids[:30], [29])]
    second = [StepEntry("a", a_ids[30:50], [0, 19]), StepEntry("b", b_ids[:10], [9])]
    assert same(engine.step(first), clean.step(first))
    used = engine.cache.used_pages()
    runtime.fail_call(_products(dtype), 6)
    with pytest.raises(runtime.KernelError, match="llmx_rt_fail_call"):
        engine.step(second)
    torch.cuda.synchronize()
    assert engine.length("a") == 30 and "b" not in engine.cache.live and engine.cache.used_pages() == used
    engine.cache.check()
    assert same(engine.step(second), clean.step(second))          # the same step again is what it is on a clean engine
    # a plain decode step fails: both requests stay where they are, and the next one is right
    session, clean_session = DecodeSession(engine, ["a", "b"]), DecodeSession(clean, ["a", "b"])
    runtime.fail_call(_products(dtype), 6)
    with pytest.raises(runtime.KernelError):
        session.step([a_ids[50], b_ids[10]])
    assert (engine.length("a"), engine.length("b")) == (50, 10)
    engine.cache.check()
    got = {}
    for t in range(8):
        toks = [a_ids[50 + t], b_ids[10 + t]]
        if t == 5:                                     # by now the session replays a recording: its launch fails
            assert session.replays()
            rec = session._rec
            real, rec._graph.replay = rec._graph.replay, lambda: (_ for _ in ()).throw(RuntimeError("replay refused"))
            with pytest.raises(RuntimeError, match="replay refused"):
                session.step(toks)
            rec._graph.replay = real
            assert (engine.length("a"), engine.length("b")) == (55, 15)
            engine.cache.check()
        out, want = session.step(toks), clean_session.step(toks)
        assert same(out, want), t
        got[("a", 50 + t)], got[("b", 10 + t)] = out[0].float().cpu().numpy(), out[1].float().cpu().numpy()
    runtime.fail_call(None)
    ops_tc.check_errors()
    worst, scale, where = helpers.compare(got, {"a": a_ids[:58], "b": b_ids[:18]}, folder, dtype == "bfloat16")
    assert worst <= tol(dtype, "D") * scale, f"largest difference {worst:.3e} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_rolled_back_goes_on_as_if_the_tokens_had_never_come(model_dirs, dtype):
    """`Engine.truncate`: the keys beyond the new length are forgotten and their pages given back; feeding the same
    tokens again gives the same logits, feeding others gives theirs."""
    import torch
    from llmx_b200.engine import StepEntry, StepError
    vocab = CONFIGS["B"][0]["vocab_size"]
    ids = helpers.random_ids(vocab, 50, seed=8)
    other = ids[:27] + helpers.random_ids(vocab, 20, seed=9)
    folder, engine = _engine(model_dirs, "B", dtype, 128)
    whole = engine.step([StepEntry("r", ids, list(range(50)))]).clone()
    pages = engine.cache.used_pages()[0]
    engine.truncate("r", 27)
    assert engine.length("r") == 27 and engine.cache.used_pages()[0] == -(-27 // 8) < pages
    engine.cache.check()
    again = engine.step([StepEntry("r", ids[27:], list(range(23)))])
    if dtype == "float32":
        assert torch.equal(again, whole[27:])
    engine.truncate("r", 27)
    got_rows = engine.step([StepEntry("r", other[27:], list(range(20)))]).float().cpu().numpy()
    got = {("r", 27 + i): got_rows[i] for i in range(20)}
    worst, scale, where = helpers.compare(got, {"r": other}, folder, dtype == "bfloat16")
    assert worst <= tol(dtype, "B") * scale, f"largest difference {worst:.3e} at {where}"
    with pytest.raises(ValueError):
        engine.truncate("r", 48)
    with pytest.raises(StepError):
        engine.truncate("nobody", 1)
    engine.end("r")
    assert engine.cache.used_pages() == [0]


@pytest.mark.parametrize("name", ["B", "D", "E"])
@pytest.mark.parametrize("dtype,kv_dtype", [("bfloat16", "float32"), ("float32", "bfloat16")])
def test_a_cache_type_of_its_own(model_dirs, name, dtype, kv_dtype):
    """The cache's element type is an option of its own (the reference's ModelOptions.kv_k / kv_v,
    src/model/runtime.hpp:80-84): bfloat16 products over a float32 cache leave only the products' rounding, float32
    products over a bfloat16 cache only the cache's.  Both run the general kernels; mixed cutting with pages used
    again, against the plain implementation rounding exactly what each rounds."""
    from llmx_b200.engine import Engine, EngineOptions
    d16, d32, page = model_dirs[name]
    folder = d32 if dtype == "float32" else d16
    vocab = CONFIGS[name][0]["vocab_size"]
    requests = {f"k{i}": helpers.random_ids(vocab, n, seed=60 + i) for i, n in enumerate([70, 9, 40, 33, 1])}
    steps = helpers.trace_mixed(requests)
    engine = Engine.from_dir(folder, EngineOptions(dtype=dtype, kv_dtype=kv_dtype, kv_tokens=helpers.tokens_needed(steps),
                                                   page_size=page, max_requests=4))
    import torch
    assert engine.cache.groups[0].storage.dtype is getattr(torch, kv_dtype)
    got = helpers.run_trace(engine, steps)
    engine.cache.check()
    worst, scale, where = helpers.compare(got, requests, folder, dtype == "bfloat16", cache=kv_dtype)
    # float32 products over a bfloat16 cache: the plain twin rounds the same keys and values, so only the order of
    # float32 sums differs -- but a key rounded on the other side of a bfloat16 step moves a logit by 1e-3 of the scale
    bound = tol("bfloat16", name) if dtype == "bfloat16" else 2e-3
    assert worst <= bound * scale, f"largest difference {worst:.3e} at {where} (logit scale {scale:.3f})"


def test_an_engine_that_is_dropped_gives_its_memory_back(model_dirs):
    """The kernels' descriptors of the cache belong to the cache (not to a module), so nothing outlives the engine:
    after `del`, the device's free memory is back where it was."""
    import gc
    import torch
    from llmx_b200.engine import Engine, EngineOptions, StepEntry
    d16, _, page = model_dirs["D"]
    warm = Engine.from_dir(d16, EngineOptions(dtype="bfloat16", kv_tokens=64, page_size=page, max_requests=2))
    warm.step([StepEntry("w", [1] * 40, [39])])            # kernels loaded, per-device buffers made
    del warm
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    before = torch.cuda.mem_get_info()[0]
    engine = Engine.from_dir(d16, EngineOptions(dtype="bfloat16", kv_tokens=512 * 1024, page_size=page, max_requests=2))
    held = engine.cache.storage_bytes()
    assert held >= 256 << 20
    engine.step([StepEntry("x", [1] * 40, [39])])
    engine.step([StepEntry("x", [2], [0])])
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] <= before - held
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    assert torch.cuda.mem_get_info()[0] >= before - (32 << 20)


@pytest.mark.parametrize("name", ["D", "wide"])
def test_invariant_schedules_give_a_row_the_same_bits_in_any_batch(model_dirs, wide_model_dir, name):
    """`EngineOptions.invariant` on the bfloat16 path: kernels and schedules follow sizes alone, so a position's logits
    are the same bits however the tokens were cut and whatever else was in the step (the reference's rule,
    src/backends/backend.hpp:141-150).  Without it the bits move with the batch; the difference is bounded."""
    import torch
    from llmx_b200.engine import Engine, EngineOptions
    if name == "wide":
        folder, page, vocab, lengths = wide_model_dir, 16, WIDE["vocab_size"], [150, 70, 33, 2]
    else:
        folder, page, vocab, lengths = model_dirs[name][0], model_dirs[name][2], CONFIGS[name][0]["vocab_size"], [70, 9, 40, 33, 133]
    requests = {f"i{i}": helpers.random_ids(vocab, n, seed=80 + i) for i, n in enumerate(lengths)}
    runs = {}
    for invariant in (True, False):
        for make in (helpers.trace_whole, helpers.trace_portions, helpers.trace_mixed):
            steps = make(requests)
            engine = Engine.from_dir(folder, EngineOptions(dtype="bfloat16", kv_tokens=helpers.tokens_needed(steps), page_size=page,
                                                           max_requests=4, invariant=invariant))
            runs[(invariant, make.__name__)] = helpers.run_trace(engine, steps)
            del engine
    base = runs[(True, "trace_whole")]
    worst, scale, where = helpers.compare(base, requests, folder, True)
    assert worst <= tol("bfloat16", name) * scale
    for make in ("trace_portions", "trace_mixed"):
        other = runs[(True, make)]
        assert all(np.array_equal(base[k], other[k]) for k in base), make
    # the serving schedules: not the same bits, but close
    moved = max(float(np.abs(runs[(False, "trace_mixed")][k] - runs[(False, "trace_whole")][k]).max()) for k in base)
    assert moved <= 1e-2 * scale


@pytest.mark.parametrize("name", ["A", "wide"])
def test_products_on_pairs_of_sms_and_on_single_blocks_agree_with_the_plain_model(model_dirs, wide_model_dir, name):
    """Prompt portions of more than 64 tokens run their output and down products on pairs of SMs
    (csrc/gemm_tc_pair.cu); with that turned off, on single blocks.  Both stay within the bfloat16 budget."""
    from llmx_b200 import runtime
    from llmx_b200.engine import Engine, EngineOptions
    if name == "wide":
        folder, page, vocab = wide_model_dir, 16, WIDE["vocab_size"]
    else:
        folder, page, vocab = model_dirs[name][0], model_dirs[name][2], CONFIGS[name][0]["vocab_size"]
    requests = {"p0": helpers.random_ids(vocab, 300, seed=91), "p1": helpers.random_ids(vocab, 131, seed=92)}
    steps = helpers.trace_whole(requests)
    for on in (True, False):
        before = runtime.pair_products(on)
        try:
            engine = Engine.from_dir(folder, EngineOptions(dtype="bfloat16", kv_tokens=helpers.tokens_needed(steps), page_size=page,
                                                           max_requests=2))
            got = helpers.run_trace(engine, steps)
            del engine
        finally:
            runtime.pair_products(before)
        worst, scale, where = helpers.compare(got, requests, folder, True)
        assert worst <= tol("bfloat16", name) * scale, (on, where)
