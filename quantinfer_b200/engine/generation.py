"""The one generation loop: prompts in, tokens out, through the scheduler.

Both entry points, the Python `Model` and the `quantinfer generate` command,
call `run_requests`; nothing else in the package loops over steps and samples.
It submits every prompt to a :class:`Scheduler` over the engine's step function
and its sampler, lets decode steps run ahead of the host where the engine
replays them from CUDA graphs, and hands the events out as they arrive.

The reference has two loops: its command line steps a session by hand
(apps/quantinfer-cli/src/commands/generate.rs:255-276) while its C binding
drives the session (bindings/c/src/lib.rs:195-252). Here both go one way, so
that prompt portions, the token budget, steps that run ahead and the policy for
a full page pool are reachable from either.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from ..errors import QuantInferError
from ..sampling.params import GenerationConfig
from .pipeline import DecodePipeline
from .scheduler import FailedEvent, Scheduler, StoppedEvent, TokenEvent


@dataclass
class RequestResult:
    prompt: list
    tokens: list = field(default_factory=list)
    stop_reason: Optional[str] = None
    first_token_at: Optional[float] = None     # time.perf_counter() when the first token reached the host
    last_token_at: Optional[float] = None


@dataclass
class GenerationRun:
    results: list                    # RequestResult, in the order of the prompts
    scheduler: Scheduler
    started_at: float
    ended_at: float

    def all_first_tokens_at(self) -> Optional[float]:
        stamps = [r.first_token_at for r in self.results]
        return None if any(s is None for s in stamps) else max(stamps)


def run_requests(engine, sampler, prompts: Sequence[Sequence[int]], configs: Sequence[GenerationConfig], *,
                 max_batch_tokens: int = 2048, chunk_size: Optional[int] = None, run_ahead: bool = True,
                 max_sequences: Optional[int] = None, timeout: Optional[float] = None,
                 on_event: Optional[Callable] = None) -> GenerationRun:
    """Generates for every prompt with its own options. A failed request raises
    QuantInferError after every request of the call has given its pages back."""
    if len(prompts) != len(configs):
        raise ValueError(f"{len(prompts)} prompts for {len(configs)} generation configs")
    cache = engine.cache
    sequences = min(max_sequences or cache.max_requests, cache.max_requests)
    pipeline = DecodePipeline(engine, sampler) if run_ahead and engine.use_graphs else None
    # the sampler reads the step's status word together with the tokens: one wait per step
    # a request's options go into its slot's record on the device when it is admitted (with the tokens it
    # has emitted, if it comes back after a preemption); sampling then reads them there
    sched = Scheduler(cache, lambda entries: engine.step(entries, check_status=False), sampler.sample_step,
                      vocab_size=engine.spec.vocab_size, max_sequences=sequences,
                      max_tokens=max(max_batch_tokens, sequences), chunk_size=chunk_size, pipeline=pipeline,
                      admit_fn=lambda r: engine.assign_sampling(r.id, r.config, len(r.emitted)))
    started = time.perf_counter()
    ids = [sched.submit(list(p), cfg, timeout=timeout) for p, cfg in zip(prompts, configs)]
    results = {rid: RequestResult(list(p)) for rid, p in zip(ids, prompts)}
    failure = None

    def book(ev):
        nonlocal failure
        now = time.perf_counter()
        res = results[ev.request_id]
        if isinstance(ev, TokenEvent):
            res.tokens.append(ev.token_id)
            res.first_token_at = res.first_token_at or now
            res.last_token_at = now
            res.stop_reason = ev.stop_reason
        elif isinstance(ev, StoppedEvent):
            res.stop_reason = ev.reason
        elif isinstance(ev, FailedEvent):
            res.stop_reason = "Failed"
            failure = failure or f"request {ev.request_id} failed: {ev.error}"
        if on_event:
            on_event(ev)

    try:
        sched.run(book)
    finally:
        for rid in ids:
            if rid in cache.requests:
                cache.close(rid)
    if failure:
        raise QuantInferError(failure)
    return GenerationRun([results[rid] for rid in ids], sched, started, time.perf_counter())
