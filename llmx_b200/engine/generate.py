"""Generation: the Python entry point.  `LLM(model_dir).generate(prompts, params)`.

The loop is the reference's generate loop run for many requests at once
(src/inference/generate.hpp:19-124 for one request; the server's rounds, docs/SERVER.md:143-227):
plan a step, run it through `Engine.step`, draw a token for every entry that asked for logits,
record it, finish and free what ended.  Token ids in, token ids out: the tokenizer is not part of
this engine.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, Iterable, List, Optional, Sequence, Union

import torch

from ..sampling import RequestSampling, SamplingParams, sample, sample_async
from .decode_loop import DecodeSession
from .engine import Engine, EngineOptions, StepEntry
from .scheduler import PlannedEntry, Request, Scheduler


@dataclass
class GenerationOutput:
    request_id: Hashable
    prompt: List[int]
    tokens: List[int]
    finish_reason: str


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    steps: int = 0
    prefill_seconds: float = 0.0     # wall time of steps that held prompt portions only
    decode_seconds: float = 0.0      # wall time of all other steps
    preemptions: int = 0


class LLM:
    """A loaded model ready to generate.

    model:            a folder with config.json and safetensors files (or an `Engine`)
    dtype:            "bfloat16" (the serving path) or "float32" (everything in true 32-bit)
    kv_tokens:        tokens the cache pool is made for (default: the model's context, at most 1/3 of free memory)
    ubatch:           the most tokens one step holds (the reference's --ubatch; its default there is 512, here 2,048: a
                      prompt of 8,192 tokens goes through in 119 ms in portions of 2,048 and in 156 ms in portions of 512)
    max_seqs:         the most requests that run at once
    reserve:          "full" or "prompt" (see llmx_b200.engine.scheduler)
    yarn, yarn_original_ctx:  the rope scaled by YaRN at this factor over this trained length (the reference's
                      --yarn and --yarn-original-ctx); the context becomes factor x length
    kv_dtype:         the cache's element type when it is not the path's ("bfloat16" or "float32"; the reference's
                      --cache-type-k / --cache-type-v)
    invariant:        schedules chosen by sizes alone, so that a request's reply does not depend on what it was
                      batched with, bit for bit (slower; see parts.base.Precision)
    """

    def __init__(self, model: Union[str, Engine], *, dtype: str = "bfloat16", kv_tokens: Optional[int] = None,
                 page_size: int = 16, ubatch: int = 2048, max_seqs: int = 16, reserve: str = "full",
                 device: str = "cuda:0", yarn: Optional[float] = None, yarn_original_ctx: Optional[int] = None,
                 kv_dtype: Optional[str] = None, invariant: bool = False):
        if isinstance(model, Engine):
            self.engine = model
        else:
            if kv_tokens is None:
                kv_tokens = self._default_kv_tokens(model, kv_dtype or dtype, page_size, device)
            self.engine = Engine.from_dir(model, EngineOptions(dtype=dtype, kv_tokens=kv_tokens, page_size=page_size,
                                                               max_requests=max_seqs, device=device, yarn=yarn,
                                                               yarn_original_ctx=yarn_original_ctx, kv_dtype=kv_dtype,
                                                               invariant=invariant))
        self.ubatch, self.max_seqs, self.reserve = int(ubatch), int(max_seqs), reserve
        self.stats = GenerationStats()
        self._next_id = 0
        self._session: Optional[DecodeSession] = None
        self._session_ids = None
        self.last_decode_h2d_bytes = 0      # metadata bytes the last recorded decode step copied to the device

    @staticmethod
    def _default_kv_tokens(model_dir: str, dtype: str, page_size: int, device: str) -> int:
        from ..registry import config_from_dir
        entry, config = config_from_dir(model_dir)
        model = entry.build(config)
        per_token = 0
        width = 2 if dtype in ("bfloat16", "bf16") else 4
        for spec in model.cache_entry_specs():
            if hasattr(spec, "kv_heads"):
                per_token += 2 * spec.kv_heads * spec.head_dim * width
        free, _ = torch.cuda.mem_get_info(torch.device(device))
        by_memory = (free // 3) // max(per_token, 1)
        tokens = int(min(model.max_positions, by_memory))
        return max(page_size, tokens // page_size * page_size)

    def _scheduler(self) -> Scheduler:
        cache = self.engine.cache
        return Scheduler(pages_needed=cache.pages_needed, total_pages=cache.total_pages(),
                         max_positions=self.engine.max_positions, max_batch_tokens=self.ubatch,
                         max_requests=min(self.max_seqs, self.engine.options.max_requests), max_queue=1 << 30,
                         reserve=self.reserve, page_size=cache.page_size, eos_ids=self.engine.model.eos_ids)

    def _run(self, entries: Sequence[PlannedEntry]) -> Optional[torch.Tensor]:
        """One step.  While the same requests decode step after step, the step is a decode session's
        (recorded once, replayed); any other step goes through `Engine.step`."""
        ids = tuple(e.request.request_id for e in entries)
        if all(len(e.tokens) == 1 and e.want_last and e.request.decoding for e in entries):
            if self._session is None or self._session_ids != ids:
                self._close_session()
                self._session, self._session_ids = DecodeSession(self.engine, ids, plain_steps=4), ids
            return self._session.step([e.tokens[0] for e in entries])
        self._close_session()
        return self.engine.step([StepEntry(e.request.request_id, e.tokens, [len(e.tokens) - 1] if e.want_last else [])
                                 for e in entries], record=True)

    def _close_session(self) -> None:
        if self._session is not None:
            self._session.close()
        self._session, self._session_ids = None, None

    def _account(self, sched: Scheduler, entries: Sequence[PlannedEntry], sampled: Dict[Hashable, int], index,
                 on_token) -> List[Request]:
        """Book a finished step: the scheduler's record, the sampling states, the statistics, the callback."""
        wanting = [e for e in entries if e.want_last]
        before = {e.request.request_id: len(e.request.output) for e in wanting}
        done = sched.complete(entries, sampled)
        self.stats.steps += 1
        for e in wanting:
            r = e.request
            if len(r.output) > before[r.request_id]:
                r.sampling.saw(r.output[-1])
                self.stats.generated_tokens += 1
                if on_token:
                    on_token(index[r.request_id], r.output[-1])
        return done

    def _burst_length(self, entries: Sequence[PlannedEntry]) -> int:
        """How many decode steps these entries can run back to back without a decision of the scheduler: none can
        reach its max_tokens before the last of them, nothing depends on pages (full reservation), and no draw
        needs the token before it on the host (no penalties).  Such steps run one ahead of the host: a step is
        enqueued with the ids the device drew for the step before, and those ids are read while it runs."""
        if self.reserve != "full" or not entries:
            return 0
        for e in entries:
            r = e.request
            if not (len(e.tokens) == 1 and e.want_last and r.decoding) or r.params.penalized:
                return 0
        return min(e.request.params.max_tokens - len(e.request.output) for e in entries) - 1

    def _decode_burst(self, sched: Scheduler, entries: Sequence[PlannedEntry], steps: int, index, on_token) -> None:
        requests = [e.request for e in entries]
        ids = tuple(r.request_id for r in requests)
        if self._session is None or self._session_ids != ids:
            self._close_session()
            self._session, self._session_ids = DecodeSession(self.engine, ids, plain_steps=4), ids
        session = self._session
        states = [r.sampling for r in requests]

        def book(live: List[Request], tokens: List[int]) -> bool:
            """The step that fed every live request's last token drew `tokens` (in the session's order)."""
            fed = [PlannedEntry(r, [r.output[-1]], True) for r in live]
            sampled = {r.request_id: tokens[requests.index(r)] for r in live}
            return bool(self._account(sched, fed, sampled, index, on_token))

        pending = None                      # the draw of the step before, not yet read
        for _ in range(steps):
            if pending is not None and not session.replays():
                if book(requests, pending.result()):          # a plain step wants its tokens on the host
                    return
                pending = None
            feed = pending.ids if pending is not None else [r.output[-1] for r in requests]
            drawn = sample_async(session.step(feed), states)
            if pending is not None and book(requests, pending.result()):
                # Some request ended with the step before; the step in flight ran it once more for nothing.
                live = [r for r in requests if r.state != "finished"]
                book(live, drawn.result())
                return
            pending = drawn
        if pending is not None:
            book(requests, pending.result())
        self.last_decode_h2d_bytes = session.h2d_bytes_per_step

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 on_token=None) -> List[GenerationOutput]:
        """Generate a reply for every prompt (lists of token ids); returns them in the prompts' order.

        `on_token(request_index, token)` (optional) is called as tokens are drawn.
        """
        if params is None:
            params = SamplingParams()
        plist = list(params) if not isinstance(params, SamplingParams) else [params] * len(prompts)
        if len(plist) != len(prompts):
            raise ValueError("one SamplingParams for all prompts, or one for each")
        sched = self._scheduler()
        eos = self.engine.model.eos_ids
        requests: List[Request] = []
        for prompt, p in zip(prompts, plist):
            r = Request(("gen", self._next_id), [int(t) for t in prompt], p)
            self._next_id += 1
            r.sampling = RequestSampling(p, eos_id=eos[0] if eos else -1)
            sched.add(r)
            requests.append(r)
        index = {r.request_id: i for i, r in enumerate(requests)}
        stats = self.stats
        stats.prompt_tokens += sum(len(r.prompt) for r in requests)
        try:
            self._loop(sched, index, on_token)
        except BaseException:
            # A step that fails leaves every request where it was (Engine.step); the call as a whole gives back what
            # its requests hold, so that the engine serves the next call.
            self._close_session()
            for r in requests:
                self.engine.end(r.request_id)
            raise
        self._close_session()
        stats.preemptions += sched.preemptions
        from .. import ops_tc
        ops_tc.check_errors()
        return [GenerationOutput(r.request_id, r.prompt, list(r.output), r.finish_reason or "unknown") for r in requests]

    def _loop(self, sched: Scheduler, index, on_token) -> None:
        """Plan, step, draw and book until every request of the call has finished."""
        stats = self.stats
        while not sched.idle:
            entries = sched.plan()
            for rid in sched.take_releases():
                self.engine.end(rid)
            if not entries:
                if sched.idle:
                    break
                raise RuntimeError("the scheduler planned an empty step while requests are waiting")
            t0 = time.perf_counter()
            burst = self._burst_length(entries)
            if burst >= 2:
                self._decode_burst(sched, entries, burst, index, on_token)
                stats.decode_seconds += time.perf_counter() - t0
                for rid in sched.take_releases():
                    self.engine.end(rid)
                continue
            logits = self._run(entries)
            sampled: Dict[Hashable, int] = {}
            wanting = [e for e in entries if e.want_last]
            if wanting:
                ids = sample(logits, [e.request.sampling for e in wanting])
                for e, t in zip(wanting, ids):
                    sampled[e.request.request_id] = t
            else:
                torch.cuda.current_stream().synchronize()
            dt = time.perf_counter() - t0
            if all(not e.request.decoding and len(e.tokens) > 1 for e in entries):
                stats.prefill_seconds += dt
            else:
                stats.decode_seconds += dt
            self._account(sched, entries, sampled, index, on_token)
            for rid in sched.take_releases():
                self.engine.end(rid)
