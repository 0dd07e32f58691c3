"""Generation through the Python entry point and the command line."""
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers
import plain_qwen3 as plain
from configs import BF16_BUDGET, CONFIGS

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _check_greedy(folder, prompt, tokens, bf16, name="A"):
    """Every generated token is the plain implementation's argmax given what came before (a near tie may
    fall either way under different rounding: two logits each within the configuration's budget; anything else
    must agree)."""
    cfg, w = plain.load_folder(folder)
    ids = list(prompt)
    for t in tokens:
        logits = plain.forward(cfg, w, ids, act_round=plain.round_bf16 if bf16 else None)[-1]
        best = int(np.argmax(logits))
        gap = 2 * BF16_BUDGET[name] if bf16 else 1e-4
        assert t == best or logits[best] - logits[t] <= gap * np.abs(logits).max(), (len(ids), t, best)
        ids.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_greedy_generation(model_dirs, name, dtype):
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    d16, d32, page = model_dirs[name]
    folder = d32 if dtype == "float32" else d16
    vocab = CONFIGS[name][0]["vocab_size"]
    prompts = [helpers.random_ids(vocab, n, seed=n) for n in (5, 17, 33)]
    llm = LLM(folder, dtype=dtype, kv_tokens=256, page_size=page, ubatch=24, max_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=16, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True))
    assert [len(o.tokens) for o in outs] == [16, 16, 16] and all(o.finish_reason == "length" for o in outs)
    for p, o in zip(prompts, outs):
        _check_greedy(folder, p, o.tokens, dtype == "bfloat16", name)
    assert llm.engine.cache.used_pages() == [0]
    assert llm.stats.generated_tokens == 48 and llm.stats.prompt_tokens == 55


def test_temperature_sampling_is_reproducible_and_independent_of_the_batch(model_dirs):
    """Four requests (prompts of 1, 9, 40 and 70 tokens) as mixed portions and decoded tokens, temperature 0.8
    with fixed seeds: the same seeds give the same replies, and a request's reply is the one it gets alone."""
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    _, folder, page = model_dirs["B"]
    vocab = CONFIGS["B"][0]["vocab_size"]
    prompts = [helpers.random_ids(vocab, n, seed=n) for n in (1, 9, 40, 70)]
    params = [SamplingParams(max_tokens=12, temp=0.8, top_k=40, top_p=0.95, seed=100 + i, ignore_eos=True) for i in range(4)]
    llm = LLM(folder, dtype="float32", kv_tokens=512, page_size=page, ubatch=32, max_seqs=4)
    first = [o.tokens for o in llm.generate(prompts, params)]
    again = [o.tokens for o in llm.generate(prompts, params)]
    assert first == again and all(len(t) == 12 for t in first)
    alone = [llm.generate([p], [q])[0].tokens for p, q in zip(prompts, params)]
    assert alone == first
    other = [o.tokens for o in llm.generate(prompts, [SamplingParams(max_tokens=12, temp=0.8, seed=7 + i, ignore_eos=True) for i in range(4)])]
    assert other != first


def test_end_of_sequence_and_length(model_dirs):
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    _, folder, page = model_dirs["A"]
    llm = LLM(folder, dtype="float32", kv_tokens=256, page_size=page)
    prompt = helpers.random_ids(256, 9, seed=1)
    greedy = llm.generate([prompt], SamplingParams(max_tokens=10, temp=0.0, ignore_eos=True))[0].tokens
    # Make the third generated token the end-of-sequence id: the reply stops before it.
    llm.engine.model.eos_ids = (greedy[2],)
    out = llm.generate([prompt], SamplingParams(max_tokens=10, temp=0.0))[0]
    stop_at = greedy.index(greedy[2])
    assert out.tokens == greedy[:stop_at] and out.finish_reason == "eos"
    masked = llm.generate([prompt], SamplingParams(max_tokens=10, temp=0.0, ignore_eos=True))[0]
    assert greedy[2] not in masked.tokens and masked.finish_reason == "length"   # masked out of the draw


def test_requests_end_at_different_steps_while_decoding_runs_ahead(model_dirs):
    """Decoding steps are enqueued one ahead of the host, which reads a step's ids while the next one runs.  A
    request that draws the end-of-sequence id is therefore seen a step late: its reply must stop where it would
    have, the others' replies must not change, and every token is handed to the callback once, in order."""
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    _, folder, page = model_dirs["A"]
    llm = LLM(folder, dtype="float32", kv_tokens=1024, page_size=page, max_seqs=4)
    llm.engine.model.eos_ids = ()
    prompts = [helpers.random_ids(256, n, seed=40 + s) for s, n in enumerate([9, 17, 5, 12])]
    limits = [30, 30, 30, 22]
    alone = [llm.generate([p], SamplingParams(max_tokens=n, temp=0.0))[0].tokens for p, n in zip(prompts, limits)]
    eos = alone[1][11]                                   # the second request ends at its twelfth token at the latest
    llm.engine.model.eos_ids = (eos,)
    want = [t[:t.index(eos)] if eos in t else t for t in alone]
    assert any(len(w) < len(a) for w, a in zip(want, alone))
    streamed = {i: [] for i in range(4)}
    outs = llm.generate(prompts, [SamplingParams(max_tokens=n, temp=0.0) for n in limits],
                        on_token=lambda i, t: streamed[i].append(t))
    for i, out in enumerate(outs):
        assert out.tokens == want[i], i
        assert out.finish_reason == ("eos" if len(want[i]) < len(alone[i]) else "length")
        assert streamed[i] == want[i]
    llm.engine.cache.check()
    assert llm.engine.cache.used_pages() == [0]


def test_pages_running_out_pauses_and_recomputes_with_the_same_replies(model_dirs):
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    _, folder, page = model_dirs["A"]
    prompts = [helpers.random_ids(256, 28, seed=s) for s in range(3)]
    params = SamplingParams(max_tokens=40, temp=0.0, ignore_eos=True)
    roomy = LLM(folder, dtype="float32", kv_tokens=512, page_size=16, ubatch=64, max_seqs=3)
    want = [o.tokens for o in roomy.generate(prompts, params)]
    tight = LLM(folder, dtype="float32", kv_tokens=96, page_size=16, ubatch=64, max_seqs=3, reserve="prompt")
    got = [o.tokens for o in tight.generate(prompts, params)]
    assert tight.stats.preemptions > 0 and got == want
    tight.engine.cache.check()
    assert tight.engine.cache.used_pages() == [0]


@pytest.mark.parametrize("reserve,kv_tokens", [("full", 640), ("prompt", 208)])
def test_random_workloads_against_each_request_alone(model_dirs, reserve, kv_tokens):
    """Rounds of random prompts, limits and end-of-sequence ids through `generate` -- with recorded steps of every
    shape that comes twice, decoding run ahead of the host, and (with the small pool) requests paused and
    recomputed -- each reply against the same request continued alone, one plain step a token."""
    import random
    import torch
    from llmx_b200.engine import Engine, EngineOptions, StepEntry
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    _, folder, _ = model_dirs["A"]
    vocab = CONFIGS["A"][0]["vocab_size"]
    rng = random.Random(5)
    ref = Engine.from_dir(folder, EngineOptions(dtype="float32", kv_tokens=256, page_size=16, max_requests=1))

    def alone(prompt, limit, eos):
        out, logits = [], ref.step([StepEntry("ref", prompt, [len(prompt) - 1])])
        while True:
            token = int(torch.argmax(logits[0]).item())
            if token == eos:
                reason = "eos"
                break
            out.append(token)
            if len(out) >= limit:
                reason = "length"
                break
            logits = ref.step([StepEntry("ref", [token], [0])])
        ref.end("ref")
        return out, reason

    engine = Engine.from_dir(folder, EngineOptions(dtype="float32", kv_tokens=kv_tokens, page_size=16, max_requests=4,
                                                   record_after=2))
    llm = LLM(engine, ubatch=48, max_seqs=4, reserve=reserve)
    for _ in range(12):
        eos = rng.randrange(vocab) if rng.random() < 0.7 else -1
        engine.model.eos_ids = (eos,) if eos >= 0 else ()
        n = rng.randrange(1, 9)
        prompts = [[rng.randrange(vocab) for _ in range(rng.randrange(1, 90))] for _ in range(n)]
        limits = [rng.randrange(1, 45) for _ in range(n)]
        streamed = {i: [] for i in range(n)}
        outs = llm.generate(prompts, [SamplingParams(max_tokens=k, temp=0.0) for k in limits],
                            on_token=lambda i, t: streamed[i].append(t))
        for i, out in enumerate(outs):
            want, reason = alone(prompts[i], limits[i], eos)
            assert (out.tokens, out.finish_reason, streamed[i]) == (want, reason, want), (i, len(prompts[i]), limits[i])
        engine.cache.check()
        assert engine.cache.used_pages() == [0]
    assert engine.decode_recordings and engine.step_recordings
    if reserve == "prompt":
        assert llm.stats.preemptions > 0


def test_command_line(model_dirs, tmp_path):
    d16, _, _ = model_dirs["D"]
    exe = [sys.executable, os.path.join(ROOT, "bin", "llmx")]
    run = subprocess.run(exe + ["generate", d16, "5,17,3,99", "-n", "6", "--temp", "0", "--ignore-eos", "--verbose"],
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = run.stdout.splitlines()
    ids = next(l for l in lines if l.startswith("ids: "))
    assert len(ids[5:].split(",")) == 6
    assert any(l.startswith("pp: 4 tok") for l in lines) and any(l.startswith("tg: 6 tok") for l in lines)
    tokens = [int(t) for t in ids[5:].split(",")]
    _check_greedy(d16, [5, 17, 3, 99], tokens, True)
    f = tmp_path / "prompt.txt"
    f.write_text("5 17 3 99")
    again = subprocess.run(exe + ["generate", d16, "--file", str(f), "-n", "6", "--temp", "0", "--ignore-eos"],
                           capture_output=True, text=True, timeout=600)
    assert again.returncode == 0 and ids in again.stdout
    # the same through the native engine: files, scheduling and draws in C++
    native = subprocess.run(exe + ["generate", d16, "5,17,3,99", "-n", "6", "--temp", "0", "--ignore-eos", "--engine", "native", "--verbose"],
                            capture_output=True, text=True, timeout=600)
    assert native.returncode == 0, native.stderr[-2000:]
    assert "pp: 4 tok" in native.stdout and "tg: 6 tok" in native.stdout and "finish length" in native.stdout
    native_ids = next(l for l in native.stdout.splitlines() if l.startswith("ids: "))
    _check_greedy(d16, [5, 17, 3, 99], [int(t) for t in native_ids[5:].split(",")], True)
    for bad in (["generate", d16, "1,2", "--temp", "-1"], ["generate", d16, "1,2", "--engine", "rust"], ["generate", d16, "1,2", "-n", "3", "-n", "4"],
                ["generate", d16], ["generate", d16, "1,2", "--bogus"], ["generate", d16, "1,2", "--topp", "1.5"],
                ["frobnicate"]):
        r = subprocess.run(exe + bad, capture_output=True, text=True, timeout=120)
        assert r.returncode == 2 and "usage:" in r.stderr, bad
    lg = subprocess.run(exe + ["logits", d16, "5,17,3,99", "--top", "3", "--last", "2"], capture_output=True, text=True, timeout=600)
    per = subprocess.run(exe + ["logits", d16, "5,17,3,99", "--top", "3", "--last", "2", "--per-token"], capture_output=True,
                         text=True, timeout=600)
    assert lg.returncode == 0 and per.returncode == 0, lg.stderr[-2000:] + per.stderr[-2000:]
    lines = [l for l in lg.stdout.splitlines() if l.startswith("pos ")]
    assert [l.split(":")[0] for l in lines] == ["pos 2 after 3", "pos 3 after 99"]
    assert int(lines[1].split(": ")[1].split(":")[0]) == tokens[0]          # the best token after the prompt is what greedy drew
    assert [l.split()[4].split(":")[0] for l in per.stdout.splitlines() if l.startswith("pos ")] == \
           [l.split()[4].split(":")[0] for l in lines]
    bench = subprocess.run(exe + ["bench", "--model", d16, "--p", "40", "--n", "5", "--r", "1", "--seqs", "2"],
                           capture_output=True, text=True, timeout=600)
    assert bench.returncode == 0 and "bench: pp40 " in bench.stdout and "bench: x2 tg5 " in bench.stdout, bench.stderr[-2000:]
    deep = subprocess.run(exe + ["bench", "--model", d16, "--p", "20", "--n", "4", "--r", "2", "--depth", "70", "--ubatch", "16",
                                 "--profile"], capture_output=True, text=True, timeout=600)
    assert deep.returncode == 0 and "bench: pp20 @ d70 " in deep.stdout and "bench: tg4 @ d70 " in deep.stdout, deep.stderr[-2000:]
    assert "profile pp20:" in deep.stdout and "profile tg:" in deep.stdout and "llmx_rmsnorm" in deep.stdout
    synthetic = subprocess.run(exe + ["bench", "--size", "96", "--iters", "2", "--p", "12", "--n", "3"], capture_output=True,
                               text=True, timeout=600)
    assert synthetic.returncode == 0, synthetic.stderr[-2000:]
    for line in ("bench: matmul 96x96", "bench: rms_norm n=96", "bench: norm_rope n=96", "bench: prefill  12 tok",
                 "bench: decode    3 tok"):
        assert line in synthetic.stdout, synthetic.stdout
    for bad in (["bench", "--r", "2"], ["bench", "--model", d16, "--size", "64"]):
        r = subprocess.run(exe + bad, capture_output=True, text=True, timeout=120)
        assert r.returncode == 2 and "usage:" in r.stderr, bad


@pytest.fixture(scope="module")
def baseline_dirs(tmp_path_factory):
    """The two tiny configurations exactly as the benchmark's baseline names them (context 128 and 256, no rope
    scaling): {name: (bfloat16 folder, float32 folder)}."""
    import torch
    from configs import BASELINE_A, BASELINE_B
    from llmx_b200.config import Qwen3Config
    from llmx_b200.weights import write_random_model
    out = {}
    for name, raw, seed in (("A", BASELINE_A, 0), ("B", BASELINE_B, 1)):
        c = Qwen3Config.from_dict(raw)
        assert c.max_position_embeddings == (128 if name == "A" else 256) and c.rope_scaling is None
        d16, d32 = str(tmp_path_factory.mktemp(f"base_{name}_bf16")), str(tmp_path_factory.mktemp(f"base_{name}_f32"))
        write_random_model(d16, c, seed, dtype=torch.bfloat16)
        write_random_model(d32, c, seed, dtype=torch.float32)
        out[name] = (d16, d32)
    return out


def test_baseline_tiny_a_workload(baseline_dirs):
    """Tiny A to the letter, float32: three requests of 5, 17 and 33 tokens, 16 greedy tokens each, against the
    plain implementation token by token."""
    from configs import BASELINE_A
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    folder = baseline_dirs["A"][1]
    prompts = [helpers.random_ids(BASELINE_A["vocab_size"], n, seed=n) for n in (5, 17, 33)]
    llm = LLM(folder, dtype="float32", kv_tokens=192, page_size=16, ubatch=24, max_seqs=3)
    assert llm.engine.max_positions == 128
    outs = llm.generate(prompts, SamplingParams(max_tokens=16, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert len(o.tokens) == 16
        _check_greedy(folder, p, o.tokens, False)
    assert llm.engine.cache.used_pages() == [0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_baseline_tiny_b_workload_on_both_storages(baseline_dirs, dtype):
    """Tiny B to the letter: four requests of 1, 9, 40 and 70 tokens as mixed portions and decoded tokens, pages of 8,
    temperature 0.8 with fixed seeds -- on the float32 check path and on bfloat16 storage.  The same seeds give the
    same replies, and a request's reply is the one it gets alone.  On bfloat16 that needs schedules that do not follow
    the batch (`invariant`): with the serving schedules a row's last bits move with the batch and a draw near a
    boundary may fall the other way."""
    from configs import BASELINE_B
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    folder = baseline_dirs["B"][1 if dtype == "float32" else 0]
    prompts = [helpers.random_ids(BASELINE_B["vocab_size"], n, seed=n) for n in (1, 9, 40, 70)]
    params = [SamplingParams(max_tokens=12, temp=0.8, top_k=40, top_p=0.95, seed=100 + i, ignore_eos=True) for i in range(4)]
    llm = LLM(folder, dtype=dtype, kv_tokens=512, page_size=8, ubatch=32, max_seqs=4, invariant=dtype == "bfloat16")
    assert llm.engine.max_positions == 256
    first = [o.tokens for o in llm.generate(prompts, params)]
    again = [o.tokens for o in llm.generate(prompts, params)]
    assert first == again and all(len(t) == 12 for t in first)
    alone = [llm.generate([p], [q])[0].tokens for p, q in zip(prompts, params)]
    assert alone == first
    # every drawn token has weight in the plain implementation's distribution (it is among its top 40)
    cfg, w = plain.load_folder(folder)
    for p, reply in zip(prompts, first):
        ids = list(p)
        for t in reply:
            logits = plain.forward(cfg, w, ids, act_round=plain.round_bf16 if dtype == "bfloat16" else None)[-1]
            assert logits[t] >= np.sort(logits)[-41]
            ids.append(t)


def test_a_call_that_fails_gives_back_what_its_requests_hold(model_dirs):
    """A step fails on the host in the middle of `generate` (prompts half fed, some requests decoding): the error
    reaches the caller, every page is back, and the same call again gives the replies of an engine that never failed."""
    from llmx_b200 import runtime
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    _, folder, page = model_dirs["A"]
    prompts = [helpers.random_ids(256, n, seed=70 + n) for n in (40, 9, 33)]
    params = SamplingParams(max_tokens=10, temp=0.0, ignore_eos=True)
    llm = LLM(folder, dtype="float32", kv_tokens=512, page_size=page, ubatch=16, max_seqs=3)
    want = [o.tokens for o in llm.generate(prompts, params)]
    runtime.fail_call("llmx_attention_plain", 7)            # the fourth step's first layer
    with pytest.raises(runtime.KernelError):
        llm.generate(prompts, params)
    runtime.fail_call(None)
    llm.engine.cache.check()
    assert llm.engine.cache.used_pages() == [0] and not llm.engine.cache.live
    assert [o.tokens for o in llm.generate(prompts, params)] == want
