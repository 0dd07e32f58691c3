"""The native runtime from a C++ program: tests/native/drive_model.cpp includes csrc/runtime/llmx_runtime.h, links
the runtime library, loads the kernel libraries from their folder and runs a tiny model -- a prompt in two
portions, then single tokens, over a paged cache of its own -- with no Python in the process.  Its logits are held
to the plain implementation, in float32 and in bfloat16."""
import os
import subprocess

import numpy as np
import pytest
import torch

import helpers
import plain_qwen3 as plain
from configs import BF16_BUDGET, CONFIGS

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _dump(folder, out_dir, dtype, ids, page, positions):
    """The model folder as raw tensors under the names the driver asks for, with q/k/v and gate/up stacked."""
    cfg, w = plain.load_folder(folder)
    cfg = plain.normalized_config(cfg)
    code = 1 if dtype == "bfloat16" else 0
    lines = []

    def put(name, array, as_code):
        t = torch.from_numpy(np.ascontiguousarray(array))
        raw = t.to(torch.bfloat16).view(torch.int16).numpy() if as_code == 1 else t.to(torch.float32).numpy()
        raw.tofile(os.path.join(out_dir, name + ".bin"))
        lines.append(f"{name} {as_code} {t.numel()} {name}.bin")

    put("embed", w["model.embed_tokens.weight"], code)
    if not cfg["tie_word_embeddings"]:
        put("head", w["lm_head.weight"], code)
    put("norm", w["model.norm.weight"], 0)
    cos, sin = plain.rope_tables(positions, cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
    put("cos", cos, 0)
    put("sin", sin, 0)
    for l in range(cfg["num_hidden_layers"]):
        p, q = f"model.layers.{l}.", f"layers.{l}."
        put(q + "qkv", np.concatenate([w[p + f"self_attn.{n}_proj.weight"] for n in "qkv"]), code)
        put(q + "o", w[p + "self_attn.o_proj.weight"], code)
        put(q + "gate_up", np.concatenate([w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]]), code)
        put(q + "down", w[p + "mlp.down_proj.weight"], code)
        put(q + "q_norm", w[p + "self_attn.q_norm.weight"], 0)
        put(q + "k_norm", w[p + "self_attn.k_norm.weight"], 0)
        put(q + "norm1", w[p + "input_layernorm.weight"], 0)
        put(q + "norm2", w[p + "post_attention_layernorm.weight"], 0)
    head = (f"{cfg['num_hidden_layers']} {cfg['hidden_size']} {cfg['num_attention_heads']} {cfg['num_key_value_heads']} "
            f"{cfg['head_dim']} {cfg['intermediate_size']} {cfg['vocab_size']} {code} {cfg['rms_norm_eps']!r} {positions} {page} "
            f"{1 if cfg['tie_word_embeddings'] else 0}\n{len(ids)}\n" + " ".join(str(t) for t in ids) + "\n")
    with open(os.path.join(out_dir, "manifest.txt"), "w") as f:
        f.write(head + "\n".join(lines) + "\n")


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    """The C++ program, compiled against the header and linked with the built runtime library."""
    from llmx_b200.csrc import build
    runtime_so = build.build("runtime")
    for name in build.LIBRARIES:           # the program cannot compile what it finds missing: everything is built first
        build.build(name)
    exe = str(tmp_path_factory.mktemp("native") / "drive_model")
    include = os.path.join(os.path.dirname(build.__file__), "runtime")
    cmd = [build._nvcc(), "-O1", "-std=c++17", "-I", include, "-o", exe, os.path.join(HERE, "native", "drive_model.cpp"),
           runtime_so, "-Xlinker", "-rpath", "-Xlinker", os.path.dirname(runtime_so)]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stdout + done.stderr
    return exe, os.path.dirname(runtime_so)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D", "E"])
def test_a_cpp_program_drives_a_model_through_the_runtimes_header(model_dirs, driver, tmp_path, name, dtype):
    exe, kernels = driver
    d16, d32, page = model_dirs[name]
    folder = d32 if dtype == "float32" else d16
    ids = helpers.random_ids(CONFIGS[name][0]["vocab_size"], 150 if name != "A" else 70, seed=17)
    dump = tmp_path / "dump"
    dump.mkdir()
    _dump(folder, str(dump), dtype, ids, page, 256)
    out = str(tmp_path / "logits.f32")
    done = subprocess.run([exe, str(dump), kernels, out], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout + done.stderr
    assert done.stdout.startswith("steps ")
    got = np.fromfile(out, dtype="<f4").reshape(len(ids), -1)
    ref = helpers.reference_logits(folder, ids, dtype == "bfloat16")
    tol = BF16_BUDGET[name] if dtype == "bfloat16" else 1e-4
    worst = float(np.abs(got - ref).max())
    assert worst <= tol * float(np.abs(ref).max()), f"largest difference {worst:.3e}"


def test_a_block_written_elsewhere_runs_inside_the_native_model(model_dirs):
    """`llmx_callback_create`: a block that is a function of another language (here a ctypes callback) takes its
    place in the native model's walk.  The callback stands in for the model's second layer and runs that layer's own
    native block on a workspace of its own, so the logits must be exactly those of the model without the detour."""
    import ctypes
    from llmx_b200 import runtime
    from llmx_b200.engine import Engine, EngineOptions, StepEntry
    folder = model_dirs["D"][1]
    engine = Engine.from_dir(folder, EngineOptions(dtype="float32", kv_tokens=128, page_size=16, max_requests=2))
    model = engine.model
    ids = helpers.random_ids(CONFIGS["D"][0]["vocab_size"], 40, seed=4)
    want = engine.step([StepEntry("w", ids, list(range(40)))]).clone()
    engine.end("w")
    assert model.native
    rt = runtime.lib()
    calls, keep = [], []
    CALLBACK = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(runtime.StepStruct), ctypes.c_int, ctypes.c_void_p,
                                ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int)

    def second_layer(user, step, kind, h, x, rows, cache_entry, write_cache):
        calls.append((kind, rows, cache_entry, write_cache))
        mine = runtime.StepStruct.from_buffer_copy(step.contents)       # the same step, a workspace of its own
        need = rt.llmx_part_workspace(model.blocks[1].native, ctypes.byref(mine), rows, cache_entry)
        ws = torch.empty(int(need), dtype=torch.uint8, device="cuda")
        keep.append(ws)
        mine.workspace, mine.workspace_bytes = ws.data_ptr(), int(need)
        return rt.llmx_block_forward(model.blocks[1].native, ctypes.byref(mine), x, rows, cache_entry, write_cache)

    fn = CALLBACK(second_layer)
    detour = rt.llmx_callback_create(0, ctypes.cast(fn, ctypes.c_void_p), None, model.embedding.hidden)
    assert detour
    blocks = (ctypes.c_void_p * 2)(model.blocks[0].native, detour)
    order = (runtime.LayerStepStruct * 2)(runtime.LayerStepStruct(0, 0, 1), runtime.LayerStepStruct(1, 1, 1))
    twin = rt.llmx_model_create(model.embedding.native, blocks, 2, order, 2, model.head.native, model.embedding.hidden, model.vocab_size)
    assert twin
    real, model._native.handle = model._native.handle, twin              # the engine's steps now walk the twin
    try:
        got = engine.step([StepEntry("c", ids[:25], list(range(25)))])
        got = torch.cat([got, engine.step([StepEntry("c", ids[25:], list(range(15)))])])
    finally:
        model._native.handle = real
        rt.llmx_model_destroy(twin)
        rt.llmx_part_destroy(detour)
    assert calls == [(0, 25, 1, 1), (0, 15, 1, 1)]
    assert torch.equal(got, want)
