"""The native engine (csrc/runtime/llmx_engine.h) through its thin Python face: the same traces and the same
generation as the Python engine, with the cache's bookkeeping, the step's metadata, the scheduler and the sampler's
state in C++."""
import numpy as np
import pytest

import helpers
from configs import CONFIGS, BF16_BUDGET, BF16_UNCALIBRATED

pytestmark = pytest.mark.gpu


def tol(dtype, name):
    return 1e-4 if dtype == "float32" else BF16_BUDGET.get(name, BF16_UNCALIBRATED)


class AsEngine:
    """The native engine behind the two calls `helpers.run_trace` makes."""

    def __init__(self, native):
        self.native, self.ids, self.next = native, {}, 1000

    def _id(self, name):
        if name not in self.ids:
            self.ids[name], self.next = self.next, self.next + 1
        return self.ids[name]

    def step(self, entries, record=False):
        import torch
        rows = self.native.forward([(self._id(e.request_id), list(e.tokens), list(e.want)) for e in entries])
        return torch.from_numpy(rows) if rows.shape[0] else None

    def end(self, name):
        self.native.end(self._id(name))
        self.ids.pop(name, None)


LENGTHS = [70, 1, 9, 40, 133, 33]


def _requests(name):
    vocab = CONFIGS[name][0]["vocab_size"]
    return {f"r{i}": helpers.random_ids(vocab, n, seed=100 * i + n) for i, n in enumerate(LENGTHS)}


def _python_engine(folder, dtype, page, kv_tokens, max_requests=4, invariant=False):
    from llmx_b200.engine import Engine, EngineOptions
    return Engine.from_dir(folder, EngineOptions(dtype=dtype, kv_tokens=kv_tokens, page_size=page, max_requests=max_requests,
                                                 invariant=invariant))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_native_engine_replays_the_traces(model_dirs, name, dtype, cutting):
    """Whole prompts, the last tokens one by one, portions of changing size, and requests mixed over so few pages that
    they are used again: the native engine's logits against the plain implementation, and its cache's books after
    every trace (no page lost, held twice or freed twice)."""
    from llmx_b200.native_engine import NativeEngine
    folder, page = model_dirs[name][0 if dtype == "bfloat16" else 1], model_dirs[name][2]
    requests = _requests(name)
    make = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_tail_decoded(r, 12), "portions": helpers.trace_portions,
            "mixed": helpers.trace_mixed}[cutting]
    steps = make(requests)
    kv_tokens = helpers.tokens_needed(steps)
    engine = _python_engine(folder, dtype, page, kv_tokens)
    native = NativeEngine.over(engine)
    got = helpers.run_trace(AsEngine(native), steps)
    native.check()
    total, free = native.pages()[0]
    assert free == total                                  # every request of a trace ends
    worst, scale, where = helpers.compare(got, requests, folder, dtype == "bfloat16")
    assert worst <= tol(dtype, name) * scale, where
    native.close()


def test_native_engine_refuses_and_rolls_back(model_dirs):
    """A batch it does not take, and pages that do not suffice: an error by name, and every request as it was."""
    from llmx_b200.native_engine import NativeEngine, NativeEngineError, ERR_CACHE, ERR_REFUSED
    folder, page = model_dirs["A"][1], model_dirs["A"][2]
    vocab = CONFIGS["A"][0]["vocab_size"]
    native = NativeEngine.over(_python_engine(folder, "float32", page, 4 * page), kv_tokens=4 * page)
    ids = helpers.random_ids(vocab, 3 * page, seed=1)
    first = native.forward([(1, ids, [len(ids) - 1])])
    for bad, text in (([(1, [vocab], [0])], "outside the vocabulary"), ([(2, [], [])], "without tokens"),
                      ([(2, [1, 2], [2])], "wanted place"), ([(2, [1], []), (2, [1], [])], "appears twice")):
        with pytest.raises(NativeEngineError) as err:
            native.forward(bad)
        assert err.value.code == ERR_REFUSED and text in str(err.value)
    with pytest.raises(NativeEngineError) as err:
        native.forward([(1, [5], [0]), (2, helpers.random_ids(vocab, 2 * page, seed=2), [])])      # request 2 cannot fit
    assert err.value.code == ERR_CACHE
    native.check()
    assert native.length(1) == len(ids) and native.length(2) == 0 and native.held_pages(1) == 3
    # the same prompt again from the start, after a roll-back: the same logits
    native.truncate(1, 0)
    assert native.held_pages(1) == 0
    again = native.forward([(1, ids, [len(ids) - 1])])
    assert np.array_equal(first, again)
    native.end(1)
    native.check()
    native.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_native_engine_generates_what_the_python_engine_generates(model_dirs, dtype):
    """add_request / step: greedy and seeded draws, prompts longer than a step's token budget, more requests than run at
    once.  The replies equal `LLM.generate`'s, which runs the same kernels under a scheduler of the same policy."""
    from llmx_b200.engine.generate import LLM
    from llmx_b200.native_engine import NativeEngine
    from llmx_b200.sampling import SamplingParams
    name = "B"
    folder, page = model_dirs[name][0 if dtype == "bfloat16" else 1], model_dirs[name][2]
    vocab = CONFIGS[name][0]["vocab_size"]
    prompts = [helpers.random_ids(vocab, n, seed=40 + n) for n in (1, 9, 40, 70, 23)]
    params = [SamplingParams(max_tokens=12, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True),
              SamplingParams(max_tokens=9, temp=0.8, top_k=20, top_p=0.9, seed=7, ignore_eos=True),
              SamplingParams(max_tokens=14, temp=1.0, top_k=0, top_p=1.0, min_p=0.05, seed=11, ignore_eos=True),
              SamplingParams(max_tokens=6, temp=0.7, penalty=1.3, presence_penalty=0.5, frequency_penalty=0.2, seed=3, ignore_eos=True),
              SamplingParams(max_tokens=10, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True)]
    # (bfloat16 with the schedules that follow sizes alone: sums added in pieces move in their last bits from run to run,
    # and a reply may part from a near tie on; those schedules give a row the same bits every time)
    engine = _python_engine(folder, dtype, page, 1024, max_requests=3, invariant=dtype == "bfloat16")
    llm = LLM(engine, ubatch=32, max_seqs=3)
    want = [(o.tokens, o.finish_reason) for o in llm.generate(prompts, params)]
    native = NativeEngine.over(engine, ubatch=32, max_requests=3)
    got = native.generate(prompts, params)
    assert got == want
    native.check()
    assert all(free == total for total, free in native.pages())
    native.close()


def test_native_engine_pauses_the_latest_request_when_pages_run_out(model_dirs):
    """Prompt-only reservation over a small pool: pages run out while decoding, the request admitted last gives its
    pages back and recomputes later, and every reply is what the request gives alone."""
    from llmx_b200.native_engine import NativeEngine
    from llmx_b200.sampling import SamplingParams
    folder, page = model_dirs["A"][1], model_dirs["A"][2]
    vocab = CONFIGS["A"][0]["vocab_size"]
    prompts = [helpers.random_ids(vocab, n, seed=60 + n) for n in (20, 25, 30)]
    p = SamplingParams(max_tokens=40, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True)
    roomy = NativeEngine.over(_python_engine(folder, "float32", page, 1024), ubatch=64)
    alone = [roomy.generate([q], p)[0] for q in prompts]
    roomy.close()
    pool = ((30 + 40 + page - 1) // page + 4) * page          # one request alone fits with a little to spare, three do not
    tight = NativeEngine.over(_python_engine(folder, "float32", page, pool), kv_tokens=pool, ubatch=64, reserve="prompt")
    got = tight.generate(prompts, p)
    assert tight.preemptions > 0
    assert got == alone
    tight.check()
    tight.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_native_loader_reads_a_model_folder(model_dirs, name, dtype):
    """`NativeEngine.load`: config.json and the safetensors file read by the native loader (its own JSON reader, its
    own rotation tables, weights stacked and converted on the host), a mixed trace against the plain implementation."""
    from llmx_b200.native_engine import NativeEngine
    folder, page = model_dirs[name][0 if dtype == "bfloat16" else 1], model_dirs[name][2]
    requests = _requests(name)
    steps = helpers.trace_mixed(requests)
    native = NativeEngine.load(folder, dtype=dtype, kv_tokens=helpers.tokens_needed(steps), page_size=page, max_requests=4)
    got = helpers.run_trace(AsEngine(native), steps)
    native.check()
    worst, scale, where = helpers.compare(got, requests, folder, dtype == "bfloat16")
    assert worst <= tol(dtype, name) * scale, where
    native.close()


def test_a_failure_that_shows_after_the_step_ran_takes_the_step_back(model_dirs):
    """A kernel that gives up a bounded wait is known only when the step's results are read, after the step's rows were
    committed to the cache.  Here the failure is made on the host: a block written in the test (a callback in the native
    model's walk) runs the model's own second layer and, when armed, writes an error code into the step's error word as
    such a kernel would.  The failing step must leave pages, lengths and the requests' generators as they were: the
    replies, drawn with temperature, equal those of an engine that never failed."""
    import ctypes
    import torch
    from cuda.bindings import runtime as cudart
    from llmx_b200 import runtime
    from llmx_b200.engine import Engine, EngineOptions
    from llmx_b200.native_engine import NativeEngine, NativeEngineError
    from llmx_b200.sampling import SamplingParams
    folder = model_dirs["D"][1]
    vocab = CONFIGS["D"][0]["vocab_size"]
    engine = Engine.from_dir(folder, EngineOptions(dtype="float32", kv_tokens=256, page_size=16, max_requests=4))
    model = engine.model
    assert model.native                                # the native model is made on first use
    rt = runtime.lib()
    armed, keep = [False], []
    CALLBACK = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(runtime.StepStruct), ctypes.c_int, ctypes.c_void_p,
                                ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int)
    code = np.array([77], dtype=np.int32)

    def second_layer(user, step, kind, h, x, rows, cache_entry, write_cache):
        mine = runtime.StepStruct.from_buffer_copy(step.contents)
        need = rt.llmx_part_workspace(model.blocks[1].native, ctypes.byref(mine), rows, cache_entry)
        ws = torch.empty(int(need), dtype=torch.uint8, device="cuda")
        keep.append(ws)
        mine.workspace, mine.workspace_bytes = ws.data_ptr(), int(need)
        if armed[0]:
            err, = cudart.cudaMemcpy(int(step.contents.error_word), code.ctypes.data, 4, cudart.cudaMemcpyKind.cudaMemcpyHostToDevice)
            assert int(err) == 0
        return rt.llmx_block_forward(model.blocks[1].native, ctypes.byref(mine), x, rows, cache_entry, write_cache)

    fn = CALLBACK(second_layer)
    detour = rt.llmx_callback_create(0, ctypes.cast(fn, ctypes.c_void_p), None, model.embedding.hidden)
    n_blocks = len(model.blocks)
    blocks = (ctypes.c_void_p * n_blocks)(*[detour if i == 1 else b.native for i, b in enumerate(model.blocks)])
    order = (runtime.LayerStepStruct * n_blocks)(*[runtime.LayerStepStruct(i, i, 1) for i in range(n_blocks)])
    twin = rt.llmx_model_create(model.embedding.native, blocks, n_blocks, order, n_blocks, model.head.native, model.embedding.hidden,
                                model.vocab_size)
    assert detour and twin
    real, model._native.handle = model._native.handle, twin
    prompts = [helpers.random_ids(vocab, 20, seed=31), helpers.random_ids(vocab, 9, seed=32)]
    params = [SamplingParams(max_tokens=7, temp=0.9, top_k=20, top_p=0.9, seed=5, ignore_eos=True),
              SamplingParams(max_tokens=5, temp=1.1, top_k=0, top_p=0.8, seed=6, ignore_eos=True)]

    def run(fail_at):
        native = NativeEngine.over(engine, kv_tokens=256, page_size=16, max_requests=4)
        native.record_steps(False)                     # the callback copies from the host, which no recording may hold
        ids = [native.add_request(p, sp) for p, sp in zip(prompts, params)]
        failures, step = 0, 0
        while not native.idle:
            if step in fail_at:
                held = [native.held_pages(i) for i in ids]
                armed[0] = True
                try:
                    with pytest.raises(NativeEngineError) as e:
                        native.step()
                finally:
                    armed[0] = False
                assert e.value.code == 20005 and "code 77" in str(e.value)
                native.check()
                assert [native.held_pages(i) for i in ids] == held
                fail_at = fail_at - {step}
                failures += 1
                continue
            native.step()
            step += 1
        out = [native.output(i) for i in ids]
        native.check()
        native.close()
        return out, failures

    try:
        want, none = run(set())
        got, failures = run({0, 1, 3})                 # the prompts' step, the first decoding step, a later one
    finally:
        model._native.handle = real
        rt.llmx_model_destroy(twin)
        rt.llmx_part_destroy(detour)
    assert none == 0 and failures == 3
    assert got == want and [len(o[0]) for o in want] == [7, 5]


def test_native_loader_reads_a_sharded_folder(model_dirs, tmp_path):
    """The same tensors in three files named by model.safetensors.index.json (and a stray file the index does not name,
    which is not read): the same logits, bit for bit, as from the single file."""
    import json
    import os
    import shutil
    from llmx_b200.native_engine import NativeEngine
    from llmx_b200.weights import TensorDirectory, write_safetensors
    name = "B"
    folder, page = model_dirs[name][1], model_dirs[name][2]
    ids = helpers.random_ids(CONFIGS[name][0]["vocab_size"], 24, seed=6)
    whole = NativeEngine.load(folder, dtype="float32", kv_tokens=128, page_size=page)
    want = whole.forward([(1, ids, list(range(len(ids))))])
    whole.close()
    d = TensorDirectory(folder)
    names = sorted(d.names())
    shards = tmp_path / "shards"
    os.makedirs(shards)
    shutil.copy(os.path.join(folder, "config.json"), shards / "config.json")
    weight_map = {}
    for k in range(3):
        part = {n: d.tensor(n).clone() for n in names[k::3]}
        fname = f"model-0000{k + 1}-of-00003.safetensors"
        write_safetensors(str(shards / fname), part)
        weight_map.update({n: fname for n in part})
    write_safetensors(str(shards / "consolidated.safetensors"), {n: d.tensor(n).clone() for n in names[:2]})
    d.close()
    (shards / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": 0}, "weight_map": weight_map}))
    sharded = NativeEngine.load(str(shards), dtype="float32", kv_tokens=128, page_size=page)
    got = sharded.forward([(1, ids, list(range(len(ids))))])
    sharded.close()
    assert np.array_equal(got, want)


def test_native_loader_converts_between_stored_and_path_types(model_dirs):
    """A bfloat16 folder run in float32 (widened exactly) and a float32 folder run in bfloat16 (rounded to nearest even):
    the same logits as the Python engine gives for the same folder and path."""
    from llmx_b200.native_engine import NativeEngine
    from llmx_b200.engine import StepEntry
    name = "A"
    vocab, page = CONFIGS[name][0]["vocab_size"], model_dirs[name][2]
    ids = helpers.random_ids(vocab, 40, seed=5)
    for folder, dtype in ((model_dirs[name][0], "float32"), (model_dirs[name][1], "bfloat16")):
        native = NativeEngine.load(folder, dtype=dtype, kv_tokens=256, page_size=page)
        got = native.forward([(1, ids, list(range(len(ids))))])
        native.close()
        engine = _python_engine(folder, dtype, page, 256)
        want = engine.step([StepEntry("a", ids, list(range(len(ids))))]).float().cpu().numpy()
        scale = np.abs(want).max()
        assert np.abs(got - want).max() <= (1e-5 if dtype == "float32" else tol(dtype, name)) * scale


def test_a_cpp_program_generates_through_the_native_engine(model_dirs, tmp_path):
    """tests/native/drive_engine.cpp: `llmx::Engine::load`, `add_request`, `step` with no Python in the process; its
    replies equal the Python engine's."""
    import os
    import subprocess
    from llmx_b200.csrc import build
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    name = "B"
    folder, page = model_dirs[name][1], model_dirs[name][2]
    vocab = CONFIGS[name][0]["vocab_size"]
    prompts = [helpers.random_ids(vocab, n, seed=70 + n) for n in (5, 33, 12)]
    llm = LLM(_python_engine(folder, "float32", page, 512), ubatch=16, max_seqs=2)
    greedy = SamplingParams(max_tokens=8, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True)
    seeded = SamplingParams(max_tokens=8, temp=0.9, top_k=10, top_p=0.9, seed=5, ignore_eos=True)
    want = [o.tokens for o in llm.generate(prompts, [greedy, seeded, greedy])]
    # every kernel library the run needs, built and in one folder
    runtime_so = build.build("runtime")
    for lib in ("rowwise", "gemm_plain", "attention_plain", "sampling"):
        build.build(lib)
    kernel_dir = os.path.dirname(runtime_so)
    here = os.path.dirname(os.path.abspath(__file__))
    exe = str(tmp_path / "drive_engine")
    include = os.path.join(os.path.dirname(build.__file__), "runtime")
    cmd = [build._nvcc(), "-O1", "-std=c++17", "-I", include, "-o", exe, os.path.join(here, "native", "drive_engine.cpp"),
           runtime_so, "-Xlinker", "-rpath", "-Xlinker", kernel_dir]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stdout + done.stderr
    lines = []
    for ids, kind in zip(prompts, ("greedy", "seeded", "greedy")):
        lines.append(kind + " " + " ".join(str(t) for t in ids))
    out = subprocess.run([exe, folder, kernel_dir, str(page)], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    got = [[int(t) for t in line.split()] for line in out.stdout.strip().splitlines()]
    assert got == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_native_engine_records_the_shapes_that_keep_coming(model_dirs, dtype):
    """Decode steps of the same requests, and the equal portions a long prompt is cut into, are recorded as CUDA graphs
    after a few plain steps and replayed: the same tokens as with recording off, and as each request gives alone."""
    from llmx_b200.native_engine import NativeEngine
    from llmx_b200.sampling import SamplingParams
    name = "D"
    folder, page = model_dirs[name][0 if dtype == "bfloat16" else 1], model_dirs[name][2]
    vocab = CONFIGS[name][0]["vocab_size"]
    prompts = [helpers.random_ids(vocab, n, seed=90 + n) for n in (400, 7, 21)]
    params = [SamplingParams(max_tokens=40, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True),
              SamplingParams(max_tokens=60, temp=0.8, top_k=30, top_p=0.95, seed=9, ignore_eos=True),
              SamplingParams(max_tokens=50, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True)]
    engine = _python_engine(folder, dtype, page, 2048, max_requests=4)
    plain = NativeEngine.over(engine, ubatch=16)
    plain.record_steps(False)
    want = plain.generate(prompts, params)
    assert plain.replays == 0
    plain.close()
    native = NativeEngine.over(engine, ubatch=16)
    got = native.generate(prompts, params)
    assert native.replays > 40                        # the decode steps, and the prompt's portions of sixteen tokens
    assert native.last_h2d_bytes < 64 * 1024
    if dtype == "float32":
        assert got == want
    else:                                             # bfloat16 sums move in their last bits from run to run; a greedy reply may part from a tie on
        assert [len(t) for t, _ in got] == [len(t) for t, _ in want]
        assert got[0][0][:8] == want[0][0][:8]
    native.check()
    # a second call finds its recordings ready
    before = native.replays
    again = native.generate(prompts[1:], params[1:])
    assert native.replays > before
    if dtype == "float32":
        assert again == want[1:]
    native.close()


def test_native_engine_runs_a_model_of_two_cache_groups_and_a_repeated_layer(tmp_path):
    """A model put together in the test from the framework's own (native) parts: a layer with rotated full attention
    that the order names twice (cache entries of its own each time), and a windowed layer without rotation or q/k norm
    that runs a second time reading the keys it wrote the first time.  The native engine keeps a pool per group, gives
    the window's pages back while the full group keeps its own, and its logits are the Python engine's bit for bit."""
    import json
    import os
    import torch
    from dataclasses import dataclass
    from llmx_b200.engine import Engine, EngineOptions
    from llmx_b200.models import LayerStep, Model
    from llmx_b200.native_engine import NativeEngine
    from llmx_b200.parts import (Attention, GatedMLP, LogitsHead, NoPositionEncoding, PreNormBlock, RMSNorm, RotaryEmbedding,
                                 TokenEmbedding)
    from llmx_b200.registry import register_architecture, unregister_architecture
    from llmx_b200.weights import RandomSource, write_safetensors

    @dataclass(frozen=True)
    class Two:
        hidden_size: int = 64
        vocab_size: int = 120
        window: int = 12

        @classmethod
        def from_dict(cls, raw):
            return cls(**{k: v for k, v in raw.items() if k not in ("architectures", "model_type")})

        def to_dict(self):
            return dict(self.__dict__, architectures=["TwoGroups"], model_type="two_groups")

    def build(cfg):
        E, H, G, D = cfg.hidden_size, 4, 2, 16
        norm = lambda: RMSNorm(E, 1e-5)          # noqa: E731
        mlp = lambda: GatedMLP(E, 96)            # noqa: E731
        blocks = [PreNormBlock(norm(), Attention(E, H, G, D, RotaryEmbedding(D, 10000.0), qk_norm_eps=1e-5), norm(), mlp()),
                  PreNormBlock(norm(), Attention(E, H, G, D, NoPositionEncoding(), qk_norm_eps=None, window=cfg.window), norm(), mlp())]
        order = [LayerStep(0, 0), LayerStep(1, 1), LayerStep(0, 2), LayerStep(1, 1, write_cache=False)]
        emb = TokenEmbedding(cfg.vocab_size, E)
        return Model(embedding=emb, blocks=blocks, head=LogitsHead(norm(), cfg.vocab_size, E, tied_to=emb), order=order,
                     vocab_size=cfg.vocab_size, max_positions=512)

    register_architecture(["TwoGroups", "two_groups"], Two, build)
    try:
        cfg = Two()
        folder = str(tmp_path)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg.to_dict(), f)
        src = RandomSource(build(cfg).tensor_specs(), 5, dtype=torch.float32, skip_optional=True)
        write_safetensors(os.path.join(folder, "model.safetensors"),
                          {n: src.tensor(n) * (4.0 if n.endswith("proj.weight") else 1.0) for n in src.names()})
        requests = {f"t{i}": helpers.random_ids(cfg.vocab_size, n, seed=i) for i, n in enumerate([50, 3, 77, 20, 1, 64])}
        for make in (helpers.trace_portions, helpers.trace_mixed):
            steps = make(requests)
            tokens = helpers.tokens_needed(steps)
            engine = Engine.from_dir(folder, EngineOptions(dtype="float32", kv_tokens=tokens, page_size=4, max_requests=4))
            assert engine.model.native and len(engine.cache.groups) == 2
            want = helpers.run_trace(engine, steps)
            native = NativeEngine.over(engine)
            got = helpers.run_trace(AsEngine(native), steps)
            native.check()
            assert all(free == total for total, free in native.pages()) and len(native.pages()) == 2
            assert all(np.array_equal(got[k], want[k]) for k in want)
            native.close()
        # the window's pages go back while the request lives; the full group's stay
        engine = Engine.from_dir(folder, EngineOptions(dtype="float32", kv_tokens=256, page_size=4, max_requests=2))
        native = NativeEngine.over(engine)
        ids = helpers.random_ids(cfg.vocab_size, 100, seed=5)
        native.forward([(1, ids[:60], [])])
        windowed = 1 if engine.cache.groups[1].spec.window else 0
        assert native.held_pages(1, 1 - windowed) == 15 and native.held_pages(1, windowed) <= 4
        for t in ids[60:]:
            native.forward([(1, [t], [0])])
            assert native.held_pages(1, windowed) <= 4
        assert native.held_pages(1, 1 - windowed) == 25
        native.close()
    finally:
        unregister_architecture(["TwoGroups", "two_groups"])
