"""The engine: a model, its cache manager, and the one step function.

`step(entries)` runs exactly the tokens it is given, as one batch, from the
cache that earlier steps left, and returns 32-bit logits at the wanted places.
Everything above it (trace replay, the scheduler, generation) goes through it.

Failure rules follow the reference's mixed batch
(crates/quantinfer-runtime/src/batch.rs:133-169 per-item checks: empty tokens,
id outside the vocabulary, over capacity; :223-242 a failed shared pass rolls
every cache back to where the step began): entries are checked on the host
before anything is launched, pages are taken for all entries or for none, and
a device status word that a kernel set (bad page, bad token) turns the step
into an error after which no request has advanced.
"""

from __future__ import annotations

from pathlib import Path
from typing import Sequence

import torch

from .. import kernels
from ..cache import CacheManager
from ..config import load_config
from ..config.spec import ModelSpec
from ..errors import KernelError, QuantInferError
from ..parts import Runtime
from ..weights.loader import load_folder
from .batch import ONLY_ON_THE_DEVICE, StepBatch, StepEntry, batch_from_packed, pack_batch
from .model import Model

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           torch.float32: torch.float32, torch.bfloat16: torch.bfloat16}

DEFAULT_PAGE_SIZE = 64
KV_BUCKET = 512   # a decode graph serves contexts up to the next multiple of this


def parse_dtype(name) -> torch.dtype:
    try:
        return _DTYPES[name]
    except KeyError:
        raise QuantInferError(f"unknown dtype {name!r}; use bfloat16 or float32") from None


class Engine:
    def __init__(self, spec: ModelSpec, tensors: dict, *, dtype="bfloat16", device="cuda:0",
                 page_size: int = DEFAULT_PAGE_SIZE, max_tokens: int | None = None,
                 num_pages: int | None = None, max_requests: int = 64, max_seq_len: int | None = None,
                 config=None, use_graphs: bool = True):
        """`tensors` are the model's weights by file name (CPU or device tensors).

        The page pool holds `num_pages` pages per layer group, or enough for
        `max_tokens` cached tokens when each request's count is rounded up to a
        multiple of 64 (or of the page size, if that is larger)."""
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is visible: the engine runs only on the GPU (there is no CPU path)")
        kernels.library()  # fail now, loudly, if the kernels cannot be built or loaded
        self.spec = spec
        self.config = config
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.runtime = Runtime(self.dtype, self.device)
        self.model = Model(spec, self.runtime)
        self.model.load(tensors)
        self.max_seq_len = min(max_seq_len or spec.max_positions, spec.max_positions)
        self.page_size = page_size
        if num_pages is None:
            if max_tokens is None:
                max_tokens = self.max_seq_len * min(max_requests, 4)
            unit = max(64, page_size)
            num_pages = -(-max_tokens // page_size)
            if unit % page_size:
                num_pages += max_requests  # pages that do not divide the rounding unit need slack
        self.cache = CacheManager(self.model.cache_needs, page_size, num_pages, max_requests,
                                  self.max_seq_len, self.dtype, self.device)
        self._views = [self.cache.view(call.cache, call.writes_cache) for call in self.model.order]
        from ..sampling.slots import RequestSlots

        self.slots = RequestSlots(max_requests, self.device)   # the sampler's record of every slot, on the device
        self.last_batch = None                                 # the device arrays of the step that ran last
        self._staging = [None, None]
        self._staging_event = [None, None]
        self._staging_turn = 0
        self.steps_run = 0
        self.use_graphs = use_graphs
        self.max_graph_batch = 64
        self._graphs = {}
        self._graph_pool = None
        self.h2d_bytes = 0
        self.h2d_bytes_max = 0

    # ---- construction ------------------------------------------------------

    @classmethod
    def from_folder(cls, folder, *, check_finite: bool = False, strict_weights: bool = False, **kw) -> "Engine":
        """The model of a folder (config.json and safetensors). `check_finite` refuses weights with
        NaN or infinities by name; `strict_weights` refuses tensors the model does not use."""
        folder = Path(folder)
        config = load_config(folder)
        spec = config.to_model_spec()
        from .model import tensor_needs_of_spec

        tensors = load_folder(folder, tensor_needs_of_spec(spec), strict=strict_weights, check_finite=check_finite)
        return cls(spec, tensors, config=config, **kw)

    # ---- requests ------------------------------------------------------------

    def open(self, request_id):
        return self.cache.open(request_id)

    def close(self, request_id) -> None:
        self.cache.close(request_id)

    def assign_sampling(self, request_id, config, emitted: int = 0) -> None:
        """Writes the sampler's record of an open request's slot (its options and the tokens it has
        emitted); `Sampler.sample_step` and the steps that run ahead draw by it."""
        self.slots.assign(self.cache.get(request_id).slot, config, emitted)

    def length(self, request_id) -> int:
        return self.cache.get(request_id).length

    # ---- the step --------------------------------------------------------------

    def _check_entries(self, entries: Sequence[StepEntry]) -> None:
        seen = set()
        vocab = self.spec.vocab_size
        for e in entries:
            if e.request_id in seen:
                raise QuantInferError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            rc = self.cache.get(e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise QuantInferError(f"request {e.request_id!r}: a step entry needs at least one token")
            for t in e.tokens:
                if not 0 <= t < vocab:
                    raise QuantInferError(f"request {e.request_id!r}: token id {t} is outside the vocabulary of {vocab}")
            if rc.length + n > self.max_seq_len:
                raise QuantInferError(
                    f"request {e.request_id!r}: {rc.length} cached + {n} new tokens exceed the limit of {self.max_seq_len} positions")
            for w in e.want:
                if not 0 <= w < n:
                    raise QuantInferError(f"request {e.request_id!r}: wanted place {w} is outside its {n} tokens")

    def _stage(self, buf):
        """Copies a packed batch into pinned host memory; returns the pinned view."""
        turn = self._staging_turn
        self._staging_turn ^= 1
        host = self._staging[turn]
        if host is None or host.numel() < buf.size:
            host = torch.empty(max(buf.size * 2, 4096), dtype=torch.int32, pin_memory=True)
            self._staging[turn] = host
            self._staging_event[turn] = torch.cuda.Event()
        else:
            self._staging_event[turn].synchronize()  # the copy that last used this buffer is done
        host[:buf.size].numpy()[:] = buf
        self.h2d_bytes = int(buf.size) * 4
        self.h2d_bytes_max = max(self.h2d_bytes_max, self.h2d_bytes)
        return host[:buf.size], self._staging_event[turn]

    def _pack(self, entries: Sequence[StepEntry]):
        reqs = [self.cache.get(e.request_id) for e in entries]
        starts = [rc.length for rc in reqs]
        slots = [rc.slot for rc in reqs]
        return (starts, slots) + pack_batch(entries, starts, slots, self.cache.host_tables, self.cache.max_blocks)

    def make_batch(self, entries: Sequence[StepEntry]) -> StepBatch:
        starts, slots, buf, layout, q_start, lens = self._pack(entries)
        host, event = self._stage(buf)
        dev = host.to(self.device, non_blocking=True)
        event.record()
        return batch_from_packed(dev, layout, entries, starts, slots, q_start, lens,
                                 len(self.cache.groups), self.cache.max_blocks)

    # ---- decode steps replayed from a CUDA graph ---------------------------------

    def _graph_eligible(self, entries) -> bool:
        return (self.use_graphs and len(entries) <= self.max_graph_batch
                and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries))

    def _graph_step(self, entries, extra_positions: int = 0, device_tokens=None):
        """A batch of single decode tokens, all wanting their logits: the packed batch has a
        fixed layout per batch size, so the forward pass is captured once per size and
        replayed; each step only copies the batch's arrays into the graph's buffer (a kernel
        reads them from the pinned buffer they were packed into). With `device_tokens`
        (int32 [entries], on the device) the token ids are taken from there instead of from
        the entries, without the host seeing them."""
        starts, slots, buf, layout, q_start, lens = self._pack(entries)
        host, event = self._stage(buf)
        b = len(entries)
        # kernels in a graph size their grids for a bound on the context, not for the
        # requests' lengths: one graph per batch size and per bucket of the longest context
        bound = min(self.max_seq_len, -(-(max(starts) + 1 + extra_positions) // KV_BUCKET) * KV_BUCKET)
        g = self._graphs.get((b, bound))
        if g is None:
            meta = torch.empty(buf.size, dtype=torch.int32, device=self.device)
            kernels.stage_step(host, meta, device_tokens)      # token_ids is the first part of the layout
            event.record()
            batch = batch_from_packed(meta, layout, entries, starts, slots, q_start, lens,
                                      len(self.cache.groups), self.cache.max_blocks)
            batch.max_kv_len = bound
            batch.extra["graph"] = True
            # a replay runs the captured kernels on whatever the device arrays then hold; host copies
            # would stay those of the capturing step, so parts get none
            batch.h_q_start = batch.h_start_pos = batch.h_kv_len = batch.h_slot_ids = ONLY_ON_THE_DEVICE
            self.last_batch = batch
            logits = self.model.forward(batch, self._views)   # eager: warms up and gives this step's result
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = kernels.launches
            with torch.cuda.graph(graph, pool=self._graph_pool):
                static_logits = self.model.forward(batch, self._views)
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            self._graphs[(b, bound)] = g = {"graph": graph, "meta": meta, "batch": batch, "logits": static_logits,
                                   "layout": layout, "launches": kernels.launches - before}
            return logits, g
        kernels.stage_step(host, g["meta"], device_tokens)
        event.record()
        self.last_batch = g["batch"]
        g["graph"].replay()
        kernels.launches += g["launches"]
        return g["logits"], g

    def step(self, entries: Sequence[StepEntry], check_status: bool = True) -> torch.Tensor:
        """Runs one batch; returns float32 logits [wanted places, vocab] on the device,
        in the order of the entries and of each entry's `want`. The tensor may be
        reused by a later step; copy what must outlive the next call."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if not entries:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        self._check_entries(entries)
        prepared = []
        try:
            for e in entries:
                self.cache.prepare(e.request_id, len(e.tokens))
                prepared.append(e.request_id)
            if self._graph_eligible(entries):
                logits, _ = self._graph_step(entries)
            else:
                batch = self.last_batch = self.make_batch(entries)
                logits = self.model.forward(batch, self._views)
            if check_status:
                self.raise_on_status()
        except Exception:
            for rid in prepared:
                self.cache.rollback(rid)
            raise
        for e in entries:
            self.cache.commit(e.request_id)
        self.steps_run += 1
        return logits

    def decode_on_device(self, request_ids, first_tokens, n_steps: int, rows, sampler) -> torch.Tensor:
        """Runs `n_steps` decode steps for the given requests without the host in the
        loop: each step's sampled tokens feed the next step on the device. `rows[i] =
        (GenerationConfig, tokens emitted so far)` as for `Sampler.sample`. Pages for all
        steps are taken first. Returns the sampled tokens, int32 [n_steps, requests]."""
        b = len(request_ids)
        entries = [StepEntry(rid, [int(t)], [0]) for rid, t in zip(request_ids, first_tokens)]
        self._check_entries(entries)
        for e in entries:
            if self.cache.get(e.request_id).length + n_steps > self.max_seq_len:
                raise QuantInferError(f"request {e.request_id!r}: {n_steps} more tokens exceed the limit of {self.max_seq_len} positions")
        prepared = []
        try:
            for e in entries:
                self.cache.prepare(e.request_id, n_steps)
                prepared.append(e.request_id)
            logits, g = self._graph_step(entries, extra_positions=n_steps - 1)   # step 0 (captures at first use)
            lay = g["layout"]

            def part(name):
                o, n = lay[name]
                return g["meta"][o:o + n]

            for rid, (cfg, emitted) in zip(request_ids, rows):
                self.assign_sampling(rid, cfg, emitted)
            greedy = all(cfg.temperature == 0.0 for cfg, _ in rows)
            batch = g["batch"]
            history = torch.empty((n_steps, b), dtype=torch.int32, device=self.device)
            tokens = torch.empty(b, dtype=torch.int32, device=self.device)
            for i in range(n_steps):
                if i:
                    g["graph"].replay()
                    kernels.launches += g["launches"]
                    logits = g["logits"]
                # the kernel finds each row's record through the step's arrays and advances its counter
                kernels.sample_slots(logits, batch.logit_rows, batch.token_req, batch.slot_ids, self.slots.table, greedy,
                                     tokens, sampler.status)
                kernels.advance_decode(part("token_ids"), part("positions"), part("start_pos"), part("kv_len"),
                                       None, tokens, history[i])
            self.raise_on_status()
        except Exception:
            for rid in prepared:
                self.cache.rollback(rid)
            raise
        for e in entries:
            self.cache.commit(e.request_id)
        self.steps_run += n_steps
        return history

    def raise_on_status(self) -> None:
        """Reads the device status word (this waits for the step) and raises if a kernel set a bit."""
        code = int(self.runtime.status.item())
        if code and kernels.knock_out:      # a measurement left kernels out: the step's results mean nothing anyway
            self.runtime.status.zero_()
            return
        if code:
            self.runtime.status.zero_()
            raise QuantInferError("the step failed on the device: " + "; ".join(kernels.status_names(code)))
