"""The scheduler: which requests run in the next step, and with which tokens.

Pure bookkeeping over plain data, so it is tested on the CPU against a fake step.  The policy
follows the reference's server scheduler (docs/SERVER.md:46-58, :136-243; src/server/policy.hpp:
153-158, :207-256; src/server/scheduler.hpp:1187-1352, :2514-2546):

  admission   first come, first served; at most `max_requests` running; a request is admitted
              when every cache group can hold what it reserves; admission stops at the first
              request that does not fit (no overtaking).
  reservation "full": prompt + max_tokens, so a running request never runs out of pages.
              "prompt": only the prompt plus one page of growth; pages may then run out while
              decoding, which is decided as follows.
  pages out   the request admitted last is paused: its pages are given back and it returns to
              the head of the line, to recompute its prompt and what it has generated when it is
              admitted again (its sampling state is kept, so its reply continues as if nothing
              happened).  A request that cannot fit even alone ends with reason "cache".
  a step      decoding requests first, one token each; then portions of prompts, in admission
              order, until the token budget of the step (`max_batch_tokens`) is spent; the portion
              that ends a prompt wants logits.
  finishing   a sampled end-of-sequence id ends the reply (the id is not part of it) unless
              ignore_eos; reaching max_tokens ends it with reason "length".
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..sampling.params import SamplingParams


@dataclass
class Request:
    request_id: Hashable
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    fed: int = 0                       # tokens of prompt + output that are in the cache
    state: str = "waiting"             # waiting | running | finished
    finish_reason: Optional[str] = None
    admissions: int = 0
    order: int = -1                    # first admission number
    sampling: object = None            # per-request sampling state, owned by the generation loop

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def decoding(self) -> bool:
        """Everything but the last sampled token is in the cache."""
        return bool(self.output) and self.fed == len(self.prompt) + len(self.output) - 1


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]
    want_last: bool


class RefusedRequest(ValueError):
    pass


class Scheduler:
    def __init__(self, *, pages_needed: Callable[[int, int], List[int]], total_pages: Sequence[int],
                 max_positions: int, max_batch_tokens: int = 512, max_requests: int = 16, max_queue: int = 64,
                 reserve: str = "full", page_size: int = 16, eos_ids: Sequence[int] = ()):
        if reserve not in ("full", "prompt"):
            raise ValueError("reserve must be 'full' or 'prompt'")
        if max_batch_tokens < 1 or max_requests < 1:
            raise ValueError("a step needs room for at least one token of one request")
        self.pages_needed = pages_needed
        self.total_pages = list(total_pages)
        self.max_positions = int(max_positions)
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_requests = int(max_requests)
        self.max_queue = int(max_queue)
        self.reserve = reserve
        self.page_size = int(page_size)
        self.eos_ids = set(eos_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self.reserved: Dict[Hashable, List[int]] = {}
        self._admission = 0
        self.preemptions = 0
        self.to_release: List[Hashable] = []     # requests whose cache the driver must give back before the next step

    # -- intake --------------------------------------------------------------------
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise RefusedRequest("generate: empty prompt")
        if len(request.prompt) + request.params.max_tokens > self.max_positions:
            raise RefusedRequest(
                f"request {request.request_id!r}: prompt of {len(request.prompt)} tokens plus max_tokens "
                f"{request.params.max_tokens} exceeds the context length of {self.max_positions}")
        alone = self.pages_needed(len(request.prompt) + request.params.max_tokens, self.max_batch_tokens)
        if any(a > t for a, t in zip(alone, self.total_pages)):
            raise RefusedRequest(
                f"request {request.request_id!r} needs {alone} pages; the cache has {self.total_pages}")
        if len(self.waiting) >= self.max_queue:
            raise RefusedRequest("the queue is full")
        self.waiting.append(request)

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # -- pages ---------------------------------------------------------------------
    def _reservation(self, r: Request) -> List[int]:
        if self.reserve == "full":
            return self.pages_needed(len(r.prompt) + r.params.max_tokens, self.max_batch_tokens)
        # What is in hand plus a page of growth.
        return self.pages_needed(len(r.tokens) + self.page_size, self.max_batch_tokens)

    def _reserved_total(self) -> List[int]:
        total = [0] * len(self.total_pages)
        for pages in self.reserved.values():
            total = [a + b for a, b in zip(total, pages)]
        return total

    def _fits(self, extra: List[int]) -> bool:
        return all(a + b <= t for a, b, t in zip(self._reserved_total(), extra, self.total_pages))

    def _admit(self) -> None:
        while self.waiting and len(self.running) < self.max_requests:
            r = self.waiting[0]
            need = self._reservation(r)
            if not self._fits(need):
                break                                   # no overtaking
            self.waiting.popleft()
            self.reserved[r.request_id] = need
            r.state = "running"
            r.fed = 0
            r.admissions += 1
            if r.order < 0:
                r.order = self._admission
                self._admission += 1
            self.running.append(r)
            self.running.sort(key=lambda q: q.order)

    def _pause_latest(self) -> Request:
        victim = max(self.running, key=lambda q: q.order)
        self.running.remove(victim)
        self.reserved.pop(victim.request_id, None)
        victim.state = "waiting"
        victim.fed = 0
        self.waiting.appendleft(victim)
        self.to_release.append(victim.request_id)
        self.preemptions += 1
        return victim

    def _grow(self) -> None:
        """Under 'prompt' reservation: make sure every running request has room for its next tokens."""
        if self.reserve == "full":
            return
        while self.running:
            short = None
            for r in sorted(self.running, key=lambda q: q.order):
                want = self.pages_needed(min(len(r.tokens) + 1, self.max_positions), self.max_batch_tokens)
                have = self.reserved[r.request_id]
                if any(w > h for w, h in zip(want, have)):
                    grown = self.pages_needed(min(len(r.tokens) + self.page_size, self.max_positions),
                                              self.max_batch_tokens)
                    extra = [max(g - h, 0) for g, h in zip(grown, have)]
                    if self._fits(extra):
                        self.reserved[r.request_id] = [max(g, h) for g, h in zip(grown, have)]
                    else:
                        short = r
                        break
            if short is None:
                return
            if len(self.running) == 1:
                # Alone and still short: it can never go on.
                r = self.running.pop()
                self.reserved.pop(r.request_id, None)
                self._finish(r, "cache")
                return
            self._pause_latest()

    # -- a step --------------------------------------------------------------------
    def plan(self) -> List[PlannedEntry]:
        self._grow()
        self._admit()
        entries: List[PlannedEntry] = []
        budget = self.max_batch_tokens
        for r in self.running:                      # decoding requests first
            if r.decoding and budget > 0:
                entries.append(PlannedEntry(r, [r.output[-1]], True))
                budget -= 1
        for r in self.running:                      # then portions of prompts, in admission order
            if r.decoding or budget <= 0:
                continue
            todo = r.tokens[r.fed:]
            if not todo:
                continue
            part = todo[:budget]
            entries.append(PlannedEntry(r, part, len(part) == len(todo)))
            budget -= len(part)
        return entries

    def _finish(self, r: Request, reason: str) -> None:
        r.state = "finished"
        r.finish_reason = reason
        self.finished.append(r)
        self.to_release.append(r.request_id)

    def complete(self, entries: Sequence[PlannedEntry], sampled: Dict[Hashable, int]) -> List[Request]:
        """Record a step: `sampled[request_id]` is the token drawn for each entry that wanted logits.
        Returns the requests that finished."""
        done: List[Request] = []
        for e in entries:
            r = e.request
            r.fed += len(e.tokens)
            if not e.want_last:
                continue
            token = sampled[r.request_id]
            stop = (token in self.eos_ids or token in r.params.stop_token_ids) and not r.params.ignore_eos
            if stop:
                reason = "eos"
            else:
                r.output.append(token)
                reason = "length" if len(r.output) >= r.params.max_tokens else None
            if reason:
                self.running.remove(r)
                self.reserved.pop(r.request_id, None)
                self._finish(r, reason)
                done.append(r)
        return done

    def take_releases(self) -> List[Hashable]:
        out, self.to_release = self.to_release, []
        return out
