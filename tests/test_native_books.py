"""The native engine's books on the CPU: its scheduler and cache bookkeeping against the Python ones, decision by
decision, under random orders of requests; and the native loader's refusals (files are checked before a device is touched)."""
import json
import os
import random
import struct

import pytest

from configs import TINY_A, TINY_B
from llmx_b200.cache.manager import CacheManager, KVSpec
from llmx_b200.engine.scheduler import Request, Scheduler
from llmx_b200.native_engine import ERR_FILE, ERR_REFUSED, ERR_WEIGHTS, NativeEngine, NativeEngineError
from llmx_b200.sampling import SamplingParams


def _python_books(specs, page, kv_tokens, window_tokens, max_requests, ubatch, reserve, eos=()):
    cache = CacheManager(specs, page, kv_tokens, max_requests, window_kv_tokens=window_tokens)
    sched = Scheduler(pages_needed=cache.pages_needed, total_pages=cache.total_pages(), max_positions=1 << 30,
                      max_batch_tokens=ubatch, max_requests=max_requests, max_queue=1 << 30, reserve=reserve,
                      page_size=page, eos_ids=eos)
    return cache, sched


def _python_step(cache, sched, draw):
    """One step of the Python scheduler over the Python cache manager with the tokens `draw` gives: the planned entries
    and what finished, as the native books report them."""
    for rid in sched.take_releases():
        if rid in cache.live:
            cache.free_request(rid)
    before = {r.request_id for r in sched.finished}
    entries = sched.plan()
    for rid in sched.take_releases():
        if rid in cache.live:
            cache.free_request(rid)
    early = [(r.request_id, -1, r.finish_reason) for r in sched.finished if r.request_id not in before]
    planned = [(e.request.request_id, len(e.tokens), e.tokens[0], e.want_last) for e in entries]
    for e in entries:
        rc = cache.live.get(e.request.request_id) or cache.new_request(e.request.request_id)
        rc.prepare(len(e.tokens))
        rc.commit()
    sampled = {e.request.request_id: draw(e.request.request_id) for e in entries if e.want_last}
    results = []
    lengths = {e.request.request_id: len(e.request.output) for e in entries}
    sched.complete(entries, sampled)
    for e in entries:
        if e.want_last:
            r = e.request
            token = sampled[r.request_id] if len(r.output) > lengths[r.request_id] else -1
            results.append((r.request_id, token, r.finish_reason))
    for rid in sched.take_releases():
        if rid in cache.live:
            cache.free_request(rid)
    return planned, early + results


def _random_run(seed, reserve):
    """Random requests (lengths, budgets, end-of-sequence draws) over two cache groups, one of them windowed, with so few
    pages that requests wait and, under prompt-only reservation, are paused: the native books plan the same entries,
    report the same results and hold the same pages as the Python scheduler and cache manager, step after step."""
    rng = random.Random(seed)
    page, kv_tokens, window_tokens = 8, 8 * 22, 8 * 18
    specs = [KVSpec(2, 16), KVSpec(2, 16, window=24), KVSpec(2, 16)]
    eos = (7,)
    cache, sched = _python_books(specs, page, kv_tokens, window_tokens, 4, 20, reserve, eos)
    native = NativeEngine.books([(2, 16, 0), (2, 16, 24), (2, 16, 0)], page_size=page, kv_tokens=kv_tokens,
                                window_kv_tokens=window_tokens, max_requests=4, ubatch=20, reserve=reserve, eos_ids=eos)
    ids = {}
    pending = []
    for k in range(14):
        prompt = [rng.randrange(8, 100) for _ in range(rng.randrange(1, 60))]
        params = SamplingParams(max_tokens=rng.randrange(1, 40), temp=0.0, ignore_eos=rng.random() < 0.3)
        pending.append((prompt, params))
    draws = random.Random(seed + 100)
    steps = 0
    while pending or not sched.idle:
        for _ in range(rng.randrange(0, 3)):                  # requests arrive while others run
            if pending:
                prompt, params = pending.pop(0)
                r = Request(len(ids), prompt, params)
                sched.add(r)
                ids[r.request_id] = native.add_request(prompt, params)
        if sched.idle:
            continue
        tokens = {}

        def draw(rid):
            tokens[rid] = 7 if draws.random() < 0.05 else draws.randrange(8, 100)
            return tokens[rid]

        want_plan, want_results = _python_step(cache, sched, draw)
        got_plan = native.plan()
        back = {v: k for k, v in ids.items()}
        assert [(back[r], n, t, w) for r, n, t, w in got_plan] == want_plan
        got_results = native.book([tokens[back[r]] for r, _, _, w in got_plan if w])
        assert [(back[r], t, f) for r, t, f in got_results] == want_results
        native.check()
        cache.check()
        assert [(t, f) for t, f in native.pages()] == list(zip(cache.total_pages(), cache.free_pages()))
        steps += 1
        assert steps < 5000
    assert native.idle
    native.plan()                                             # gives back what the last requests held
    assert all(free == total for total, free in native.pages())
    assert native.preemptions == sched.preemptions
    native.close()
    return sched.preemptions


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("reserve", ["full", "prompt"])
def test_native_books_decide_as_the_python_scheduler_and_lose_no_page(seed, reserve):
    _random_run(seed, reserve)


def test_the_random_orders_do_pause_requests():
    """The runs above are worth something only if pages do run out in some of them."""
    assert sum(_random_run(seed, "prompt") for seed in range(6)) > 0


def test_native_books_refuse_what_the_scheduler_refuses():
    native = NativeEngine.books([(2, 16, 0)], page_size=8, kv_tokens=64, max_requests=2, ubatch=8, max_positions=100, max_queue=2)
    for prompt, params, text in (([], SamplingParams(max_tokens=4), "empty prompt"),
                                 ([1] * 90, SamplingParams(max_tokens=20), "exceeds the context length"),
                                 ([1] * 60, SamplingParams(max_tokens=20), "pages of group 0")):
        with pytest.raises(NativeEngineError) as e:
            native.add_request(prompt, params)
        assert e.value.code == ERR_REFUSED and text in str(e.value)
    native.add_request([1, 2], SamplingParams(max_tokens=2))
    native.add_request([1, 2], SamplingParams(max_tokens=2))
    with pytest.raises(NativeEngineError) as e:
        native.add_request([1, 2], SamplingParams(max_tokens=2))
    assert "queue is full" in str(e.value)
    with pytest.raises(NativeEngineError) as e:
        native.book([1])
    assert "no planned step" in str(e.value)
    assert len(native.plan()) == 2
    with pytest.raises(NativeEngineError) as e:
        native.plan()
    assert "waiting for llmx_engine_book" in str(e.value)
    with pytest.raises(NativeEngineError) as e:
        native.book([1])
    assert "wants 2 tokens" in str(e.value)
    native.close()


# ---- the native loader's refusals -------------------------------------------------------------------------------------
def _folder(tmp_path, config, tensors=None, raw_file=None):
    os.makedirs(tmp_path, exist_ok=True)
    if config is not None:
        (tmp_path / "config.json").write_text(config if isinstance(config, str) else json.dumps(config))
    if raw_file is not None:
        (tmp_path / "model.safetensors").write_bytes(raw_file)
    elif tensors is not None:
        from llmx_b200.weights import write_safetensors
        write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    return str(tmp_path)


def _load_error(folder):
    with pytest.raises(NativeEngineError) as e:
        NativeEngine.load(folder, dtype="float32")
    return e.value


@pytest.mark.parametrize("change,message", [
    (dict(bogus_key=1), "unknown config.json key(s): bogus_key"),
    (dict(num_hidden_layers=0), "num_hidden_layers must be an integer >= 1"),
    (dict(hidden_size=64.5), "hidden_size must be an integer"),
    (dict(num_attention_heads=True), "num_attention_heads must be an integer"),
    (dict(num_key_value_heads=3), "divisible by KV head count"),
    (dict(head_dim=15), "head_dim must be even"),
    (dict(attention_bias=True), "attention_bias must be one of"),
    (dict(hidden_act="gelu"), "hidden_act must be one of"),
    (dict(layer_types=["full_attention", "sliding_attention"]), "every entry of layer_types"),
    (dict(rope_theta="big"), "rope_theta must be a finite number"),
    (dict(rope_scaling={"factor": 2.0}), "gives no rope_type"),
    (dict(rope_scaling={"rope_type": "linear", "factor": 2.0}), "is not supported"),
    (dict(rope_scaling={"rope_type": "yarn"}), "gives no factor"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 1.0}), "factor must be above 1"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 2.0, "mscale": 1.0}), "mscale is not supported"),
    (dict(architectures=["LlamaForCausalLM"], model_type="llama"), "no such architecture is registered"),
    (dict(tie_word_embeddings="yes"), "tie_word_embeddings must be true or false"),
    (dict(eos_token_id="two"), "eos_token_id must be an integer"),
])
def test_native_loader_reads_config_json_as_strictly(tmp_path, change, message):
    raw = dict(TINY_A)
    raw.update(change)
    err = _load_error(_folder(tmp_path, raw))
    assert err.code == ERR_FILE and message in str(err)


def test_native_loader_names_what_is_wrong_with_the_files(tmp_path):
    assert "no config.json" in str(_load_error(_folder(tmp_path / "a", None)))
    assert "not JSON" in str(_load_error(_folder(tmp_path / "b", "{not json")))
    assert "repeats the key" in str(_load_error(_folder(tmp_path / "c", '{"hidden_size": 1, "hidden_size": 2}')))
    assert "must hold an object" in str(_load_error(_folder(tmp_path / "d", "[1]")))
    missing = dict(TINY_A)
    del missing["vocab_size"], missing["hidden_size"]
    assert "missing config.json key(s): hidden_size, vocab_size" in str(_load_error(_folder(tmp_path / "e", missing)))
    assert "neither model.safetensors nor model.safetensors.index.json" in str(_load_error(_folder(tmp_path / "f", TINY_A)))

    def raw(header, data=b""):
        text = json.dumps(header).encode() if not isinstance(header, bytes) else header
        return struct.pack("<Q", len(text)) + text + data

    for k, (blob, text) in enumerate([
            (b"abc", "shorter than a safetensors header"),
            (struct.pack("<Q", 1 << 40), "exceeds"),
            (struct.pack("<Q", 100) + b"{}", "past the end"),
            (raw(b"[1, 2]"), "not a JSON object"),
            (raw(b"{not json"), "not JSON"),
            (raw({"a": {"dtype": "F32", "shape": [1]}}), "exactly dtype, shape and data_offsets"),
            (raw({"a": {"dtype": "F99", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4), "unsupported dtype"),
            (raw({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4), "offsets span"),
            (raw({"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8), "a gap between tensors"),
            (raw({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}, "b": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8), "overlap"),
            (raw({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 9), "does not end at the end of the file")]):
        err = _load_error(_folder(tmp_path / f"s{k}", TINY_A, raw_file=blob))
        assert err.code == ERR_FILE and text in str(err), (text, str(err))


def test_native_loader_follows_the_index_of_a_sharded_folder(tmp_path):
    """model.safetensors.index.json: only the files it names are read, each must hold exactly the tensors the index
    gives it, and none may lie outside the folder (src/format/safetensors.hpp:133-171).  The errors, without a GPU."""
    import torch
    from llmx_b200.weights import write_safetensors

    def folder(k, weight_map, text=None):
        d = tmp_path / f"i{k}"
        os.makedirs(d)
        (d / "config.json").write_text(json.dumps(TINY_A))
        write_safetensors(str(d / "one.safetensors"), {"a": torch.ones(2)})
        write_safetensors(str(d / "two.safetensors"), {"b": torch.zeros(3)})
        (d / "model.safetensors.index.json").write_text(text if text is not None else json.dumps({"weight_map": weight_map}))
        return str(d)

    for k, (weight_map, text, message) in enumerate([
            (None, "{not json", "not JSON"),
            (None, json.dumps({"metadata": {}}), "weight_map must map tensor names to file names"),
            ({"a": 3}, None, "weight_map must map tensor names to file names"),
            ({"a": "../one.safetensors"}, None, "outside the model folder"),
            ({"a": "sub/one.safetensors"}, None, "outside the model folder"),
            ({"a": "one.safetensors", "b": "one.safetensors"}, None, "weight_map and one.safetensors disagree on b"),
            ({"a": "one.safetensors", "b": "two.safetensors", "c": "two.safetensors"}, None, "weight_map and two.safetensors disagree on c"),
            ({"a": "one.safetensors", "b": "three.safetensors"}, None, "three.safetensors: cannot be opened")]):
        err = _load_error(folder(k, weight_map, text))
        assert err.code == ERR_FILE and message in str(err), (message, str(err))
    # A well-formed index: the files are read, and the model's comparison then names what the architecture misses.
    err = _load_error(folder("ok", {"a": "one.safetensors", "b": "two.safetensors"}))
    assert err.code == ERR_WEIGHTS and "unexpected (2)" in str(err)


def test_native_loader_lists_missing_unexpected_and_wrong_tensors_in_one_error(tmp_path):
    import torch
    from llmx_b200.config import Qwen3Config
    from llmx_b200.weights import TensorDirectory, write_random_model, write_safetensors
    good = str(tmp_path / "good")
    write_random_model(good, Qwen3Config.from_dict(TINY_B), 1, dtype=torch.float32)
    d = TensorDirectory(good)
    tensors = {n: d.tensor(n).clone() for n in d.names()}
    d.close()
    del tensors["model.layers.1.mlp.up_proj.weight"], tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(4)
    tensors["model.layers.2.self_attn.k_norm.weight"] = torch.zeros(5)
    tensors["model.embed_tokens.weight"] = tensors["model.embed_tokens.weight"].to(torch.int32)
    bad = tmp_path / "bad"
    os.makedirs(bad)
    (bad / "config.json").write_text(open(os.path.join(good, "config.json")).read())
    write_safetensors(str(bad / "model.safetensors"), tensors)
    err = _load_error(str(bad))
    text = str(err)
    assert err.code == ERR_WEIGHTS
    for part in ("missing (2)", "model.layers.1.mlp.up_proj.weight", "model.norm.weight", "unexpected (1)", "q_proj.bias",
                 "wrong (2)", "k_norm.weight: shape [5], expected [32]", "embed_tokens.weight: type I32"):
        assert part in text, part
