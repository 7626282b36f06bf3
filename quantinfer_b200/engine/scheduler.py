"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes one token per running request per step, finishes and frees.

What it keeps of the reference's `DecodeScheduler` and `DecodeSession`
(crates/quantinfer-runtime/src/scheduler.rs, session.rs): ids from 1 upward
(scheduler.rs:133-137); cache capacity reserved at admission for prompt +
max_new_tokens (scheduler.rs:120-124, session.rs:90-98), so a running request
never runs out of pages; first-come order; one decode token per request per
step; a deadline checked before and after the indivisible step
(scheduler.rs:27-45,68-73); `cancel` (scheduler.rs:145-156); the stop reasons
Eos (the token is emitted, then the request stops), MaxTokens, Cancelled,
TimedOut, Failed (session.rs:38-44,153-164) and the event shapes
(scheduler.rs:11-25). A failed step fails every request in it and none is
retried (session.rs:140-144).

What differs: the reference never splits a prompt (a prompt above the budget
runs alone and whole, scheduler.rs:192-197); here a prompt is cut into portions
so that a step never exceeds `max_tokens`, and a request that does not fit the
free pages *waits* instead of being refused (refused only if it can never fit).

When pages run out: with reservation that cannot happen to a running request.
If the step function still reports OutOfPages (the cache is shared with a user
outside this scheduler), the most recently admitted request is preempted: its
pages go back, and it returns to the head of the waiting queue with its prompt
extended by the tokens it has emitted, to be recomputed; the step is planned
again. Its sampler stream continues (the counter is the number of emitted
tokens), so its output does not change.

Running ahead: with a `pipeline` (an object with `launch(request_ids, tokens,
rows, prev)` that returns a pending result with `result()` and `discard()`),
steps whose entries are all decode tokens are launched without waiting for the
tokens of the step before, as long as the same requests go on: the device feeds
its own sampled tokens into the next step, and the host reads them one step
late. A request that ends on an EOS it could not foresee has then run one step
too many; that step's token for it is dropped. A step is never launched ahead
for a request whose pending token is its last by `max_new_tokens`, nor when
another request waits to be admitted or is still in its prompt.

The scheduler is host code over three callables and needs no device:
`step_fn(entries) -> logits`, `sample_fn(logits, [(config, emitted)]) -> tokens`,
and a :class:`CacheManager` for admission and for open/close.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional

from ..errors import OutOfPages
from ..sampling.params import GenerationConfig
from .batch import StepEntry

EOS, MAX_TOKENS, CANCELLED, TIMED_OUT, FAILED = "Eos", "MaxTokens", "Cancelled", "TimedOut", "Failed"


@dataclass
class TokenEvent:
    request_id: int
    token_id: int
    stop_reason: Optional[str] = None


@dataclass
class StoppedEvent:
    request_id: int
    reason: str


@dataclass
class FailedEvent:
    request_id: int
    error: str


@dataclass
class Request:
    id: int
    prompt: list
    config: GenerationConfig
    deadline: Optional[float] = None
    cached: int = 0                 # tokens of `prompt` already in the cache
    emitted: list = field(default_factory=list)
    carried: int = 0                # emitted tokens that a preemption moved into `prompt`
    next_token: Optional[int] = None
    stop_reason: Optional[str] = None
    reserved_pages: int = 0

    @property
    def prefilling(self) -> bool:
        return self.cached < len(self.prompt)

    def total_length(self) -> int:
        return len(self.prompt) - self.carried + self.config.max_new_tokens


class Scheduler:
    def __init__(self, cache, step_fn: Callable, sample_fn: Callable, *, vocab_size: int,
                 max_sequences: int = 8, max_tokens: int = 512, chunk_size: Optional[int] = None,
                 clock: Callable[[], float] = time.monotonic, pipeline=None, admit_fn: Optional[Callable] = None):
        """Defaults 8 sequences and 512 tokens per step are those the reference's
        server drives its scheduler with (apps/quantinfer-server/src/config.rs:32-45)."""
        if max_sequences <= 0 or max_tokens <= 0:
            raise ValueError("scheduler quotas must be positive")
        if max_sequences > max_tokens:
            raise ValueError("the token budget must cover one decode token per sequence")
        self.cache = cache
        self.step_fn = step_fn
        self.sample_fn = sample_fn
        self.vocab_size = vocab_size
        self.max_sequences = min(max_sequences, cache.max_requests)
        self.max_tokens = max_tokens
        self.chunk_size = chunk_size or max_tokens
        self.clock = clock
        self.waiting: deque = deque()
        self.running: list = []          # in admission order
        self.next_id = 1
        self.reserved_pages = 0
        self.steps = 0
        self.preemptions = 0
        self._hold_admission = False   # set by a preemption until some request gives pages back
        self.pipeline = pipeline
        self.admit_fn = admit_fn       # called with a request when it has been given its slot and its pages' reservation
        self._inflight = None          # (requests, pending result) of a launched decode step
        self.steps_ahead = 0           # steps launched before the tokens of the step before were read

    # ---- submission --------------------------------------------------------

    def submit(self, prompt, config: GenerationConfig = GenerationConfig(), timeout: Optional[float] = None) -> int:
        config.validate(self.vocab_size)
        prompt = list(prompt)
        if not prompt:
            raise ValueError("a request needs a non-empty prompt")
        for t in prompt:
            if not 0 <= t < self.vocab_size:
                raise ValueError("prompt token id is outside the model vocabulary")
        total = len(prompt) + config.max_new_tokens
        if total > self.cache.max_seq_len:
            raise ValueError("prompt and max_new_tokens exceed the maximum sequence length")
        if self.cache.pages_for(total) > self.cache.num_pages:
            raise ValueError("scheduler KV quota exceeded: the request can never fit the page pool")
        rid = self.next_id
        self.next_id += 1
        deadline = None if timeout is None else self.clock() + timeout
        self.waiting.append(Request(rid, prompt, config, deadline))
        return rid

    def cancel(self, request_id: int):
        for q in (self.waiting, self.running):
            for r in list(q):
                if r.id == request_id:
                    q.remove(r)
                    self._release(r, was_running=q is self.running)
                    r.stop_reason = CANCELLED
                    return StoppedEvent(request_id, CANCELLED)
        return None

    def pending_requests(self) -> int:
        return len(self.waiting) + len(self.running)

    # ---- decisions -----------------------------------------------------------

    def _admit(self) -> None:
        """First come, first served: the head of the queue enters when a sequence
        slot is free and the unreserved pages cover its whole length."""
        if self._hold_admission and self.running:
            return
        while self.waiting and len(self.running) < self.max_sequences:
            r = self.waiting[0]
            need = self.cache.pages_for(r.total_length())
            if self.reserved_pages + need > self.cache.num_pages:
                break
            self.waiting.popleft()
            r.reserved_pages = need
            self.reserved_pages += need
            self.cache.open(r.id)
            if self.admit_fn is not None:
                self.admit_fn(r)
            self.running.append(r)

    def plan(self) -> list:
        """The next step's entries: a decode token for every running request that
        has finished its prompt, then prompt portions in admission order while
        the budget lasts. Returns [(request, tokens, wants_logits)]."""
        self._admit()
        budget = self.max_tokens
        plan = []
        for r in self.running:
            if not r.prefilling and r.next_token is not None:
                plan.append((r, [r.next_token], True))
                budget -= 1
        for r in self.running:
            if budget <= 0:
                break
            if r.prefilling:
                n = min(len(r.prompt) - r.cached, budget, self.chunk_size)
                tokens = r.prompt[r.cached:r.cached + n]
                plan.append((r, tokens, r.cached + n == len(r.prompt)))
                budget -= n
        return plan

    # ---- one step --------------------------------------------------------------

    def step(self) -> list:
        """Plans and runs one step; returns the events it produced."""
        events = []
        now = self.clock()
        for r in list(self.running) + list(self.waiting):
            if r.deadline is not None and now >= r.deadline:
                events.append(self._stop(r, TIMED_OUT))
        if self._inflight is not None:
            events += self._resolve()
            if events or self._inflight is not None:
                return events
        while True:
            plan = self.plan()
            if not plan:
                return events
            if self.pipeline is not None and all(not r.prefilling for r, _, _ in plan):
                reqs = [r for r, _, _ in plan]
                pending = self._launch(reqs, None)
                if pending is not None:
                    self._inflight = (reqs, pending)
                    self.steps += 1
                    return events + self._resolve()
            entries = [StepEntry(r.id, tokens, [len(tokens) - 1] if want else []) for r, tokens, want in plan]
            try:
                logits = self.step_fn(entries)
                break
            except OutOfPages:
                if len(self.running) <= 1:
                    for r, _, _ in plan:
                        events.append(self._fail(r, "the page pool cannot hold this request"))
                    return events
                self._preempt(self.running[-1])
            except Exception as exc:  # a failed step fails every request in it; none is retried
                for r, _, _ in plan:
                    events.append(self._fail(r, str(exc)))
                return events
        self.steps += 1
        wanting = [(r, tokens) for r, tokens, want in plan if want]
        try:
            sampled = self.sample_fn(logits, [(r.config, len(r.emitted)) for r, _ in wanting])
        except Exception as exc:
            for r, _, _ in plan:
                events.append(self._fail(r, str(exc)))
            return events
        for r, tokens, want in plan:
            r.cached += len(tokens) if r.prefilling else 0
        return events + self._take([r for r, _ in wanting], sampled)

    def _take(self, reqs, sampled) -> list:
        """Books one sampled token for each request that is still running."""
        events = []
        now = self.clock()
        for r, token in zip(reqs, sampled):
            if r.stop_reason is not None or r not in self.running:
                continue            # ended meanwhile: the token of a step that ran ahead is dropped
            if r.deadline is not None and now >= r.deadline:
                events.append(self._stop(r, TIMED_OUT))
                continue
            token = int(token)
            r.emitted.append(token)
            if r.config.eos_token_id is not None and token == r.config.eos_token_id:
                reason = EOS
            elif len(r.emitted) == r.config.max_new_tokens:
                reason = MAX_TOKENS
            else:
                reason = None
            if reason is None:
                r.next_token = token
                events.append(TokenEvent(r.id, token, None))
            else:
                self._finish(r, reason)
                events.append(TokenEvent(r.id, token, reason))
        return events

    # ---- decode steps that run ahead ------------------------------------------------

    def _launch(self, reqs, prev):
        """Launches a decode step for `reqs` through the pipeline; None if it does not take it."""
        ahead = 0 if prev is None else 1
        rows = [(r.config, len(r.emitted) + ahead) for r in reqs]
        tokens = None if prev is not None else [r.next_token for r in reqs]
        try:
            return self.pipeline.launch([r.id for r in reqs], tokens, rows, prev)
        except OutOfPages:
            return None             # the ordinary path decides what to do about it

    def _may_run_ahead(self, reqs) -> bool:
        self._admit()
        return (len(self.running) == len(reqs) and all(a is b for a, b in zip(self.running, reqs))
                and all(not r.prefilling and len(r.emitted) + 1 < r.config.max_new_tokens for r in reqs))

    def _resolve(self) -> list:
        """Reads the tokens of the step in flight, after launching the next one if the same
        requests are sure to go on (short of an EOS)."""
        reqs, pending = self._inflight
        self._inflight = None
        ahead = None
        if self._may_run_ahead(reqs):
            try:
                ahead = self._launch(reqs, pending)
            except Exception as exc:
                pending.discard()
                return [self._fail(r, str(exc)) for r in reqs if r in self.running]
        try:
            sampled = pending.result()
        except Exception as exc:
            if ahead is not None:
                ahead.discard()
            return [self._fail(r, str(exc)) for r in reqs if r in self.running]
        events = self._take(reqs, sampled)
        if ahead is not None:
            if any(r in self.running for r in reqs):
                self._inflight = (reqs, ahead)
                self.steps += 1
                self.steps_ahead += 1
            else:
                ahead.discard()
        return events

    def run(self, on_event: Optional[Callable] = None) -> list:
        """Steps until no request is left; returns all events."""
        out = []
        while self.pending_requests():
            events = self.step()
            if not events and not self.running and self.waiting:
                # nothing runs and the head cannot be admitted: it never will be
                r = self.waiting.popleft()
                events = [self._fail(r, "the request does not fit the page pool", queued=True)]
            for e in events:
                if on_event:
                    on_event(e)
            out += events
        return out

    # ---- endings ---------------------------------------------------------------

    def _release(self, r: Request, was_running: bool) -> None:
        if was_running:
            self.cache.close(r.id)
            self.reserved_pages -= r.reserved_pages
            r.reserved_pages = 0
            self._hold_admission = False

    def _finish(self, r: Request, reason: str) -> None:
        r.stop_reason = reason
        r.next_token = None
        if r in self.running:
            self.running.remove(r)
            self._release(r, True)
        elif r in self.waiting:
            self.waiting.remove(r)

    def _stop(self, r: Request, reason: str) -> StoppedEvent:
        self._finish(r, reason)
        return StoppedEvent(r.id, reason)

    def _fail(self, r: Request, error: str, queued: bool = False) -> FailedEvent:
        if not queued:
            self._finish(r, FAILED)
        r.stop_reason = FAILED
        return FailedEvent(r.id, error)

    def _preempt(self, r: Request) -> None:
        """Gives back everything `r` holds and queues it again, first in line, with
        the tokens it has emitted appended to its prompt."""
        self.running.remove(r)
        self._release(r, True)
        new = r.emitted[r.carried:]
        r.prompt = r.prompt + new
        r.carried += len(new)
        r.cached = 0
        r.next_token = None
        self.waiting.appendleft(r)
        self.preemptions += 1
        self._hold_admission = True
