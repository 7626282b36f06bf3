"""The scheduler's decisions with a fake step function (no GPU): admission, the token
budget and prompt portions, decoding, finishing and freeing, deadlines, cancelling, and
what happens when pages run out."""

import pytest

from quantinfer_b200.cache import CacheManager, PagedKVNeed
from quantinfer_b200.engine.scheduler import (CANCELLED, EOS, MAX_TOKENS, TIMED_OUT, FailedEvent,
                                              Scheduler, StoppedEvent, TokenEvent)
from quantinfer_b200.errors import OutOfPages
from quantinfer_b200.sampling import GenerationConfig

VOCAB = 50


class FakeModel:
    """Logits put all weight on (last token + 1) % VOCAB, like the reference's `Increment`
    fake (crates/quantinfer-runtime/src/scheduler.rs:242-379). Records every batch."""

    def __init__(self, cache, fail_at=None, out_of_pages_at=()):
        self.cache = cache
        self.batches = []
        self.fail_at = fail_at
        self.out_of_pages_at = set(out_of_pages_at)
        self.calls = 0

    def step(self, entries):
        self.calls += 1
        if self.calls in self.out_of_pages_at:
            raise OutOfPages("no pages (injected)")
        if self.fail_at == self.calls:
            raise RuntimeError("injected failure")
        for e in entries:
            self.cache.prepare(e.request_id, len(e.tokens))
            self.cache.commit(e.request_id)
        self.batches.append([(e.request_id, len(e.tokens), bool(e.want)) for e in entries])
        return [(e.tokens[-1] + 1) % VOCAB for e in entries if e.want]

    def sample(self, logits, rows):
        assert len(logits) == len(rows)
        return list(logits)


def _sched(num_pages=64, page_size=4, max_requests=8, max_seq_len=256, **kw):
    cache = CacheManager([PagedKVNeed(1, 4)], page_size, num_pages, max_requests, max_seq_len, device=None)
    model = FakeModel(cache, kw.pop("fail_at", None), kw.pop("out_of_pages_at", ()))
    s = Scheduler(cache, model.step, model.sample, vocab_size=VOCAB, **kw)
    return s, model, cache


def _tokens(events, rid):
    return [e.token_id for e in events if isinstance(e, TokenEvent) and e.request_id == rid]


def test_one_request_counts_up_and_frees():
    s, model, cache = _sched()
    rid = s.submit([1, 2, 3], GenerationConfig(max_new_tokens=5))
    events = s.run()
    assert rid == 1 and _tokens(events, rid) == [4, 5, 6, 7, 8]
    assert events[-1].stop_reason == MAX_TOKENS
    assert not cache.requests and cache.free_pages() == 64 and s.reserved_pages == 0
    # one forward per emitted token: the last token is never fed back
    assert model.batches == [[(1, 3, True)]] + [[(1, 1, True)]] * 4


def test_eos_is_emitted_then_stops():
    s, model, _ = _sched()
    rid = s.submit([7], GenerationConfig(max_new_tokens=10, eos_token_id=10))
    events = s.run()
    assert _tokens(events, rid) == [8, 9, 10] and events[-1].stop_reason == EOS


def test_prompt_is_cut_into_portions_under_the_budget():
    s, model, _ = _sched(max_tokens=8, max_sequences=4)
    s.submit(list(range(20)), GenerationConfig(max_new_tokens=2))
    s.run()
    assert [b[0][1] for b in model.batches[:3]] == [8, 8, 4]
    assert [b[0][2] for b in model.batches[:3]] == [False, False, True]   # logits only when the prompt ends


def test_decodes_ride_beside_portions_and_budget_holds():
    s, model, _ = _sched(max_tokens=10, max_sequences=4, chunk_size=6)
    a = s.submit([1, 2], GenerationConfig(max_new_tokens=6))
    s.step()                                   # a's prompt
    b = s.submit(list(range(15)), GenerationConfig(max_new_tokens=2))
    events = s.run()
    assert all(sum(n for _, n, _ in batch) <= 10 for batch in model.batches)
    mixed = [batch for batch in model.batches if len(batch) == 2]
    assert mixed and mixed[0] == [(a, 1, True), (b, 6, False)]          # decode token first, then the portion
    assert _tokens(events, b) == [15, 16]


def test_admission_waits_for_pages_then_proceeds():
    s, model, cache = _sched(num_pages=6, page_size=4)    # 24 positions in all
    a = s.submit([1] * 8, GenerationConfig(max_new_tokens=8))     # 4 pages
    b = s.submit([2] * 8, GenerationConfig(max_new_tokens=8))     # 4 pages: must wait
    events = s.step()
    assert [r.id for r in s.running] == [a] and [r.id for r in s.waiting] == [b]
    events += s.run()
    assert len(_tokens(events, a)) == 8 and len(_tokens(events, b)) == 8
    first_b = next(i for i, batch in enumerate(model.batches) if any(r == b for r, _, _ in batch))
    last_a = max(i for i, batch in enumerate(model.batches) if any(r == a for r, _, _ in batch))
    assert first_b > last_a and cache.free_pages() == 6


def test_a_request_that_can_never_fit_is_refused():
    s, _, _ = _sched(num_pages=4, page_size=4)
    with pytest.raises(ValueError, match="never fit"):
        s.submit([1] * 10, GenerationConfig(max_new_tokens=10))
    with pytest.raises(ValueError, match="maximum sequence length"):
        s.submit([1] * 250, GenerationConfig(max_new_tokens=10))
    with pytest.raises(ValueError, match="outside the model vocabulary"):
        s.submit([VOCAB], GenerationConfig())
    with pytest.raises(ValueError, match="non-empty"):
        s.submit([], GenerationConfig())
    with pytest.raises(ValueError, match="max_new_tokens"):
        s.submit([1], GenerationConfig(max_new_tokens=0))


def test_out_of_pages_preempts_the_newest_and_recomputes():
    s, model, cache = _sched(out_of_pages_at={4})
    a = s.submit([1, 2, 3], GenerationConfig(max_new_tokens=6))
    b = s.submit([20, 21], GenerationConfig(max_new_tokens=6))
    events = s.run()
    assert s.preemptions == 1
    assert _tokens(events, a) == [4, 5, 6, 7, 8, 9] and _tokens(events, b) == [22, 23, 24, 25, 26, 27]
    # b came back with its emitted tokens as part of the prompt
    assert any(r == b and n > 2 and want for batch in model.batches for r, n, want in batch)
    assert not cache.requests and cache.free_pages() == 64


def test_failed_step_fails_its_requests_and_frees():
    s, model, cache = _sched(fail_at=2)
    a = s.submit([1], GenerationConfig(max_new_tokens=4))
    events = s.run()
    assert any(isinstance(e, FailedEvent) and e.request_id == a and "injected" in e.error for e in events)
    assert _tokens(events, a) == [2] and not cache.requests and s.pending_requests() == 0


def test_cancel_and_deadline():
    now = [0.0]
    s, model, cache = _sched(clock=lambda: now[0])
    a = s.submit([1], GenerationConfig(max_new_tokens=50))
    b = s.submit([5], GenerationConfig(max_new_tokens=50), timeout=10.0)
    s.step()
    ev = s.cancel(a)
    assert isinstance(ev, StoppedEvent) and ev.reason == CANCELLED and s.cancel(a) is None
    now[0] = 11.0
    events = s.step()
    assert any(isinstance(e, StoppedEvent) and e.request_id == b and e.reason == TIMED_OUT for e in events)
    assert not cache.requests and s.pending_requests() == 0
    c = s.submit([5], GenerationConfig(max_new_tokens=3), timeout=0.0)   # already past its deadline
    events = s.run()
    assert [type(e) for e in events] == [StoppedEvent] and events[0].reason == TIMED_OUT


def test_sequence_limit_and_first_come_order():
    s, model, _ = _sched(max_sequences=2, max_tokens=16)
    ids = [s.submit([i], GenerationConfig(max_new_tokens=3)) for i in range(4)]
    s.run()
    assert all(len(batch) <= 2 for batch in model.batches)
    first_seen = []
    for batch in model.batches:
        for r, _, _ in batch:
            if r not in first_seen:
                first_seen.append(r)
    assert first_seen == ids


# ---- decode steps that run ahead of the host ------------------------------------------------------


class FakePending:
    def __init__(self, values, fail=False):
        self.values, self.fail, self.read, self.dropped = values, fail, False, False

    def result(self):
        self.read = True
        if self.fail:
            raise RuntimeError("injected device failure")
        return list(self.values)

    def discard(self):
        self.dropped = True


class FakePipeline:
    """The pipeline's contract over the fake model: a launch with `prev` feeds the tokens the step
    before produced, which the scheduler has not yet seen."""

    def __init__(self, cache, fail_at=None, out_of_pages_at=(), limit=8):
        self.cache, self.fail_at, self.out_of_pages_at, self.limit = cache, fail_at, set(out_of_pages_at), limit
        self.launches = []          # (request ids, ran ahead?)
        self.rows = []
        self.pendings = []

    def launch(self, request_ids, tokens, rows, prev=None):
        if len(request_ids) > self.limit:
            return None
        if len(self.launches) + 1 in self.out_of_pages_at:
            self.out_of_pages_at.discard(len(self.launches) + 1)
            raise OutOfPages("no pages (injected)")
        feed = prev.values if prev is not None else tokens
        assert prev is None or not prev.read, "a step ran ahead of a result that was already read"
        assert len(feed) == len(request_ids) == len(rows)
        for rid in request_ids:
            self.cache.prepare(rid, 1)
            self.cache.commit(rid)
        self.launches.append((list(request_ids), prev is not None))
        self.rows.append([emitted for _, emitted in rows])
        p = FakePending([(t + 1) % VOCAB for t in feed], fail=self.fail_at == len(self.launches))
        self.pendings.append(p)
        return p


def _piped(num_pages=64, page_size=4, max_requests=8, max_seq_len=256, **kw):
    cache = CacheManager([PagedKVNeed(1, 4)], page_size, num_pages, max_requests, max_seq_len, device=None)
    model = FakeModel(cache)
    pipe = FakePipeline(cache, kw.pop("fail_at", None), kw.pop("pipe_out_of_pages_at", ()), kw.pop("limit", 8))
    s = Scheduler(cache, model.step, model.sample, vocab_size=VOCAB, pipeline=pipe, **kw)
    return s, model, pipe, cache


def test_run_ahead_gives_the_same_tokens_and_never_feeds_the_last_one():
    s, model, pipe, cache = _piped()
    rid = s.submit([1, 2, 3], GenerationConfig(max_new_tokens=6))
    events = s.run()
    assert _tokens(events, rid) == [4, 5, 6, 7, 8, 9] and events[-1].stop_reason == MAX_TOKENS
    assert model.batches == [[(1, 3, True)]]                   # the prompt; every decode step went through the pipeline
    assert pipe.launches == [([1], False)] + [([1], True)] * 4   # five decode steps for six tokens
    assert pipe.rows == [[1], [2], [3], [4], [5]]              # the sampler's counter: tokens emitted before the draw
    assert s.steps_ahead == 4 and not cache.requests and cache.free_pages() == 64 and s.reserved_pages == 0


def test_run_ahead_drops_the_step_after_an_unforeseen_eos():
    s, model, pipe, cache = _piped()
    a = s.submit([7], GenerationConfig(max_new_tokens=10, eos_token_id=11))      # 8 9 10 11(eos)
    b = s.submit([20], GenerationConfig(max_new_tokens=8))
    events = s.run()
    assert _tokens(events, a) == [8, 9, 10, 11] and _tokens(events, b) == list(range(21, 29))
    assert [e.stop_reason for e in events if isinstance(e, TokenEvent) and e.request_id == a][-1] == EOS
    # one step held a after its EOS (launched before the EOS was read); then b went on alone
    with_a = [ids for ids, _ in pipe.launches if a in ids]
    assert len(with_a) == 4 and pipe.launches[len(with_a)] == ([b], False)
    assert not cache.requests and cache.free_pages() == 64 and s.reserved_pages == 0


def test_run_ahead_stops_for_admission_and_resumes():
    s, model, pipe, cache = _piped(num_pages=6, page_size=4)
    a = s.submit([1] * 8, GenerationConfig(max_new_tokens=8))
    b = s.submit([2] * 8, GenerationConfig(max_new_tokens=8))     # waits for a's pages
    events = s.run()
    assert _tokens(events, a) == list(range(2, 10)) and _tokens(events, b) == list(range(3, 11))
    assert cache.free_pages() == 6 and s.steps_ahead > 0
    # a request that arrives while steps run ahead is admitted, and no step runs ahead while it is in its prompt
    s, model, pipe, cache = _piped(max_tokens=8, max_sequences=4)
    a = s.submit([1], GenerationConfig(max_new_tokens=12))
    ev = s.step() + s.step() + s.step()
    assert s._inflight is not None
    c = s.submit(list(range(10, 30)), GenerationConfig(max_new_tokens=3))
    ev += s.run()
    assert _tokens(ev, a) == list(range(2, 14)) and _tokens(ev, c) == [30, 31, 32]
    mixed = [batch for batch in model.batches if len(batch) == 2]
    assert mixed and all(batch[0] == (a, 1, True) for batch in mixed)
    assert not cache.requests and s.reserved_pages == 0


def test_run_ahead_with_cancel_deadline_and_failure():
    now = [0.0]
    s, model, pipe, cache = _piped(clock=lambda: now[0])
    a = s.submit([1], GenerationConfig(max_new_tokens=50))
    b = s.submit([5], GenerationConfig(max_new_tokens=50), timeout=10.0)
    s.step(); s.step(); s.step()
    assert s._inflight is not None
    assert s.cancel(a).reason == CANCELLED
    ev = s.step()                                  # the step in flight still holds a: its token for a is dropped
    assert _tokens(ev, a) == [] and len(_tokens(ev, b)) == 1
    now[0] = 11.0
    ev = s.step()
    assert any(isinstance(e, StoppedEvent) and e.request_id == b and e.reason == TIMED_OUT for e in ev)
    assert s.run() == [] and not cache.requests and s.pending_requests() == 0 and s.reserved_pages == 0
    # a step that failed on the device fails its requests; the step launched after it is dropped
    s, model, pipe, cache = _piped(fail_at=3)
    a = s.submit([1], GenerationConfig(max_new_tokens=9))
    ev = s.run()
    assert _tokens(ev, a) == [2, 3, 4] and any(isinstance(e, FailedEvent) and "injected" in e.error for e in ev)
    assert pipe.pendings[3].dropped and not cache.requests and s.pending_requests() == 0 and s.reserved_pages == 0


def test_run_ahead_falls_back_when_the_pipeline_declines():
    s, model, pipe, cache = _piped(limit=1, max_sequences=4)
    ids = [s.submit([i], GenerationConfig(max_new_tokens=4)) for i in (1, 2)]
    ev = s.run()
    assert [_tokens(ev, r) for r in ids] == [[2, 3, 4, 5], [3, 4, 5, 6]] and pipe.launches == []
    # out of pages in a launch: the ordinary path takes the step and decides
    s, model, pipe, cache = _piped(pipe_out_of_pages_at={2})
    a = s.submit([1], GenerationConfig(max_new_tokens=6))
    ev = s.run()
    assert _tokens(ev, a) == [2, 3, 4, 5, 6, 7] and not cache.requests


def test_run_ahead_equals_the_plain_scheduler_on_random_work():
    import random
    for seed in range(30):
        rng = random.Random(seed)
        work = [([rng.randrange(VOCAB) for _ in range(rng.randint(1, 12))],
                 GenerationConfig(max_new_tokens=rng.randint(1, 12),
                                  eos_token_id=rng.choice([None, None, rng.randrange(VOCAB)])),
                 rng.randint(0, 6)) for _ in range(rng.randint(1, 7))]
        results = []
        for piped in (False, True):
            kw = dict(num_pages=16, page_size=4, max_tokens=8, max_sequences=3)
            if piped:
                s, model, pipe, cache = _piped(**kw)
            else:
                s, model, cache = _sched(**kw)
            todo = sorted(work, key=lambda w: w[2])
            events, t = [], 0
            while todo or s.pending_requests():
                while todo and todo[0][2] <= t:
                    prompt, cfg, _ = todo.pop(0)
                    s.submit(prompt, cfg)
                events += s.step()
                t += 1
                assert t < 500
            cache.check_invariants()
            assert not cache.requests and cache.free_pages() == 16 and s.reserved_pages == 0
            results.append({rid: (_tokens(events, rid), [e.stop_reason for e in events
                                                          if isinstance(e, TokenEvent) and e.request_id == rid][-1])
                            for rid in range(1, len(work) + 1)})
        assert results[0] == results[1], seed
