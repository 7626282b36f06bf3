"""Decode steps that run one ahead of the host.

A decode step needs the host only to learn whether a request has ended. So the
scheduler may launch step N+1 before it has read the tokens of step N: the
sampled tokens stay on the device and feed the next step there, and their copy
to the host is read one step late. The device then never waits for the host's
bookkeeping between two decode steps.

`DecodePipeline.launch(request_ids, tokens, rows, prev)` runs one step for
requests that each bring exactly one token and returns a `PendingTokens`; its
`result()` waits for that step's copy and gives the sampled token ids (and
raises if a kernel set the status word). With `prev` (the pending result of the
step before, for the same requests in the same order) the token ids come from
the device and `tokens` is ignored.

Everything is ordered by the one stream the engine works on: the copy of step
N's tokens to the host is enqueued before step N+1's sampling overwrites them,
and a page that the host frees after reading step N is written by its next
owner only after step N+1's stray write to it.

The reference's scheduler reads every token before it plans the next step
(crates/quantinfer-runtime/src/scheduler.rs:199-231); this has no counterpart
there.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import kernels
from ..errors import QuantInferError
from .batch import StepEntry


class PendingTokens:
    """The sampled tokens of a launched step: on the device now, on the host after `result()`."""

    def __init__(self, n: int, device_tokens: torch.Tensor, host: torch.Tensor, event, status: torch.Tensor):
        self.n = n
        self.device_tokens = device_tokens
        self._host = host
        self._event = event
        self._status = status
        self._done = False

    def result(self) -> list:
        """Waits for the step; returns its token ids. Raises if a kernel set the status word."""
        self._event.synchronize()
        self._done = True
        values = self._host[:1 + self.n].tolist()
        if values[0]:
            self._status.zero_()
            raise QuantInferError(f"the step failed on the device (status {values[0]}: "
                                  + "; ".join(kernels.status_names(values[0])) + ")")
        return values[1:]

    def discard(self) -> None:
        """Waits for the step and drops what it produced, a set status word included."""
        if not self._done:
            self._event.synchronize()
            self._done = True
            if int(self._host[0]):
                self._status.zero_()


class DecodePipeline:
    def __init__(self, engine, sampler):
        if sampler.io is None or sampler.io.data_ptr() != engine.runtime.io.data_ptr():
            raise QuantInferError("the pipeline needs a sampler made by Sampler.for_engine for this engine")
        self.engine = engine
        self.sampler = sampler
        self._host = [None, None]
        self._events = [None, None]
        self._turn = 0

    def max_batch(self) -> int:
        return min(self.engine.max_graph_batch, self.sampler.io.numel() - 1) if self.engine.use_graphs else 0

    def launch(self, request_ids: Sequence, tokens: Optional[Sequence[int]], rows: Sequence[tuple],
               prev: Optional[PendingTokens] = None) -> Optional[PendingTokens]:
        """One decode step for `request_ids`; `rows[i] = (GenerationConfig, tokens emitted
        when this step's token is drawn)`. Returns None, having changed nothing, if this
        batch is not one the pipeline takes (too many requests)."""
        eng = self.engine
        b = len(request_ids)
        if b == 0 or b > self.max_batch():
            return None
        if prev is not None and prev.n != b:
            raise QuantInferError("a step that runs ahead must have the requests of the step before")
        io = self.sampler.io
        feed = [0] * b if prev is not None else [int(t) for t in tokens]
        entries = [StepEntry(rid, [t], [0]) for rid, t in zip(request_ids, feed)]
        eng._check_entries(entries)
        prepared = []
        try:
            for rid in request_ids:
                eng.cache.prepare(rid, 1)
                prepared.append(rid)
            logits, g = eng._graph_step(entries, device_tokens=None if prev is None else prev.device_tokens)
            out = io[1:1 + b]
            # the options and the draw counter come from the requests' slot records, which the device
            # advances itself: a step that runs ahead needs nothing from the host for its draw
            batch = g["batch"]
            kernels.sample_slots(logits, batch.logit_rows, batch.token_req, batch.slot_ids, eng.slots.table,
                                 all(cfg.temperature == 0.0 for cfg, _ in rows), out, self.sampler.status)
            turn = self._turn
            self._turn ^= 1
            if self._host[turn] is None:
                self._host[turn] = torch.empty(io.numel(), dtype=torch.int32, pin_memory=True)
                self._events[turn] = torch.cuda.Event()
            host, event = self._host[turn], self._events[turn]
            kernels.publish(io, host, 1 + b)
            event.record()
        except Exception:
            for rid in prepared:
                eng.cache.rollback(rid)
            raise
        # the positions are taken whatever the tokens turn out to be; a step that failed on
        # the device fails its requests, which gives everything back
        for rid in request_ids:
            eng.cache.commit(rid)
        eng.steps_run += 1
        return PendingTokens(b, out, host, event, self.sampler.status)
