"""The scheduler's decisions against a fake step: admission, portions under the token budget, decoding,
finishing and freeing, and what happens when pages run out."""
import pytest

from llmx_b200.cache import CacheManager, KVSpec
from llmx_b200.engine.scheduler import RefusedRequest, Request, Scheduler
from llmx_b200.sampling import SamplingParams

EOS = 7


def make(kv_tokens=256, page=16, budget=32, max_requests=4, reserve="full", max_positions=4096):
    cache = CacheManager([KVSpec(1, 8)], page_size=page, kv_tokens=kv_tokens, max_requests=64)
    sched = Scheduler(pages_needed=cache.pages_needed, total_pages=cache.total_pages(), max_positions=max_positions,
                      max_batch_tokens=budget, max_requests=max_requests, reserve=reserve, page_size=page, eos_ids=[EOS])
    return cache, sched


def req(rid, n_prompt, max_tokens=8, **kw):
    return Request(rid, list(range(100, 100 + n_prompt)), SamplingParams(max_tokens=max_tokens, temp=0.0, top_k=0, top_p=1.0, **kw))


class FakeEngine:
    """Holds pages like the engine does and 'samples' a fixed token (or what `answers` says)."""

    def __init__(self, cache, answers=None):
        self.cache, self.answers, self.steps = cache, answers or {}, []

    def run(self, sched, max_steps=10_000):
        while not sched.idle and max_steps:
            max_steps -= 1
            entries = sched.plan()
            for rid in sched.take_releases():
                self.cache.free_request(rid)
            if not entries and sched.idle:
                break
            assert entries, "an empty step while requests are waiting"
            assert sum(len(e.tokens) for e in entries) <= sched.max_batch_tokens
            assert len({e.request.request_id for e in entries}) == len(entries)
            sampled = {}
            for e in entries:
                rc = self.cache.live.get(e.request.request_id) or self.cache.new_request(e.request.request_id)
                assert rc.length == e.request.fed, "the scheduler and the cache disagree on what is in the cache"
                assert e.tokens == e.request.tokens[rc.length:rc.length + len(e.tokens)]
                rc.prepare(len(e.tokens))          # raises CacheExhausted if the scheduler let pages run out
                rc.commit()
                if e.want_last:
                    n = len(e.request.output)
                    sampled[e.request.request_id] = self.answers.get((e.request.request_id, n), 50 + n)
            self.steps.append([(e.request.request_id, len(e.tokens), e.want_last) for e in entries])
            sched.complete(entries, sampled)
            for rid in sched.take_releases():
                self.cache.free_request(rid)
            self.cache.check()
        assert sched.idle


def test_prompt_is_cut_into_portions_under_the_budget_then_decoded():
    cache, sched = make(budget=32)
    r = req("a", 70, max_tokens=3)
    sched.add(r)
    eng = FakeEngine(cache)
    eng.run(sched)
    assert eng.steps[:3] == [[("a", 32, False)], [("a", 32, False)], [("a", 6, True)]]
    assert eng.steps[3:] == [[("a", 1, True)], [("a", 1, True)]]
    assert r.output == [50, 51, 52] and r.finish_reason == "length" and r.state == "finished"
    assert cache.used_pages() == [0]


def test_decoding_requests_come_first_and_prompts_share_what_is_left():
    cache, sched = make(budget=16)
    sched.add(req("a", 4, max_tokens=6))
    sched.add(req("b", 40, max_tokens=2))
    eng = FakeEngine(cache)
    eng.run(sched)
    # Step 0: a's prompt (4) and 12 tokens of b.  From then on a decodes one token beside b's portions.
    assert eng.steps[0] == [("a", 4, True), ("b", 12, False)]
    assert eng.steps[1] == [("a", 1, True), ("b", 15, False)]
    assert eng.steps[2] == [("a", 1, True), ("b", 13, True)]
    assert eng.steps[3] == [("a", 1, True), ("b", 1, True)]


def test_eos_ends_a_reply_without_being_part_of_it_unless_ignored():
    cache, sched = make()
    a, b = req("a", 3, max_tokens=8), req("b", 3, max_tokens=4, ignore_eos=True)
    sched.add(a)
    sched.add(b)
    FakeEngine(cache, {("a", 2): EOS, ("b", 1): EOS}).run(sched)
    assert a.output == [50, 51] and a.finish_reason == "eos"
    assert b.output == [50, EOS, 52, 53] and b.finish_reason == "length"


def test_admission_is_first_come_first_served_and_stops_at_the_first_misfit():
    cache, sched = make(kv_tokens=128, page=16, budget=64, reserve="full")     # 8 pages
    sched.add(req("big", 60, max_tokens=20))      # 5 pages
    sched.add(req("wide", 50, max_tokens=14))     # 4 pages: does not fit beside big
    sched.add(req("small", 5, max_tokens=5))      # 1 page: would fit, but may not overtake
    entries = sched.plan()
    assert [e.request.request_id for e in entries] == ["big"]
    assert [r.request_id for r in sched.waiting] == ["wide", "small"]
    eng = FakeEngine(cache)
    sched.complete(entries, {"big": 50})
    for e in entries:                              # mirror the step in the cache, then run on
        rc = cache.new_request("big")
        rc.prepare(60)
        rc.commit()
    eng.run(sched)
    order = [s[0][0] for s in eng.steps if s]
    assert order.index("wide") < len(order) and all(r.state == "finished" for r in sched.finished)
    first_wide = next(i for i, s in enumerate(eng.steps) if any(x[0] == "wide" for x in s))
    first_small = next(i for i, s in enumerate(eng.steps) if any(x[0] == "small" for x in s))
    assert first_wide <= first_small


def test_running_requests_are_limited():
    cache, sched = make(max_requests=2, kv_tokens=1024)
    for i in range(5):
        sched.add(req(i, 4, max_tokens=3))
    eng = FakeEngine(cache)
    eng.run(sched)
    assert max(len(s) for s in eng.steps) == 2 and len(sched.finished) == 5


def test_refusals():
    cache, sched = make(kv_tokens=64, max_positions=100)
    with pytest.raises(RefusedRequest, match="empty prompt"):
        sched.add(req("e", 0))
    with pytest.raises(RefusedRequest, match="context length"):
        sched.add(req("long", 95, max_tokens=10))
    with pytest.raises(RefusedRequest, match="the cache has"):
        sched.add(req("fat", 60, max_tokens=30))
    _, tight = make()
    tight.max_queue = 1
    tight.add(req("x", 3))
    with pytest.raises(RefusedRequest, match="queue is full"):
        tight.add(req("y", 3))


def test_full_reservation_never_runs_out_of_pages():
    cache, sched = make(kv_tokens=160, page=16, budget=48, reserve="full")
    for i in range(6):
        sched.add(req(i, 20 + 7 * i, max_tokens=25))
    eng = FakeEngine(cache)
    eng.run(sched)                                 # FakeEngine.prepare would raise if pages ran out
    assert sched.preemptions == 0 and len(sched.finished) == 6
    assert all(r.finish_reason == "length" and len(r.output) == 25 for r in sched.finished)
    assert cache.used_pages() == [0]


def test_when_pages_run_out_the_latest_request_is_paused_and_recomputes():
    """Reservation of the prompt only: everyone is admitted, then decoding outgrows the pool.  The request
    admitted last gives its pages back, waits at the head of the line, recomputes its prompt and what it
    had generated, and its reply is the one it would have given undisturbed."""
    cache, sched = make(kv_tokens=96, page=16, budget=64, reserve="prompt")       # 6 pages
    rs = [req(i, 28, max_tokens=40) for i in range(3)]     # 2 pages each at admission, up to 5 each by the end
    for r in rs:
        sched.add(r)
    eng = FakeEngine(cache)
    eng.run(sched)
    assert sched.preemptions > 0
    assert all(r.finish_reason == "length" and r.output == [50 + n for n in range(40)] for r in rs)
    assert rs[0].admissions == 1 and max(r.admissions for r in rs[1:]) > 1   # the first admitted is never the one paused
    recomputed = [s for s in eng.steps if any(n > 28 for rid, n, _ in s)]
    assert recomputed, "the paused request should feed prompt and generated tokens again in one portion"
    assert cache.used_pages() == [0]


def test_a_request_that_cannot_fit_even_alone_ends_with_reason_cache():
    cache, sched = make(kv_tokens=64, page=16, budget=64, reserve="prompt")
    r = req("a", 30, max_tokens=34)                # admitted: 64 tokens are exactly the pool...
    sched.add(r)
    sched.total_pages = [3]                        # ...but the pool then turns out smaller (3 pages = 48 tokens)
    FakeEngine(cache).run(sched)
    assert r.finish_reason == "cache" and 0 < len(r.output) < 34


def test_step_layout_and_room():
    """Where a step's metadata lies in its buffer, and the room a recorded step leaves for context."""
    import numpy as np
    from llmx_b200.engine.engine import StepLayout, room_for
    lay = StepLayout([3, 1, 5], wanted=2, max_pages=[4, 2], streams=2, plan_ints=5)
    assert (lay.requests, lay.rows, lay.starts) == (3, 9, [0, 3, 4])
    # tokens, positions (two streams), row -> request, first row, rows, history, state slots read, wanted rows,
    # state slots written, then tables and slots of two cache groups, then the parts' launch plans
    assert lay.sizes == [9, 18, 9, 3, 3, 3, 3, 2, 3, 12, 9, 6, 9, 5]
    assert lay.tables(np.zeros(lay.total, dtype=np.int32), 1).shape == (3, 2) and lay.plan(np.zeros(lay.total)).size == 5
    # sections do not overlap, start on 16-byte boundaries and fill the buffer
    ends = [o + max(s, 1) for o, s in zip(lay.offsets, lay.sizes)]
    assert all(o % 4 == 0 for o in lay.offsets)
    assert all(e <= nxt for e, nxt in zip(ends, lay.offsets[1:] + [lay.total]))
    buf = np.arange(lay.total, dtype=np.int32)
    assert lay.section(buf, 3).tolist() == list(range(lay.offsets[3], lay.offsets[3] + 3))
    # an empty section (nothing wanted) still has a place of its own
    assert StepLayout([2], wanted=0, max_pages=[1]).sizes[7] == 0
    # room: a multiple of 2,048 at least one multiple ahead, never beyond what the model can address
    assert room_for(1, 1 << 20) == 4096 and room_for(2047, 1 << 20) == 4096 and room_for(2048, 1 << 20) == 6144
    assert room_for(8193, 1 << 20) == 12288 and room_for(8193, 9000) == 9000
