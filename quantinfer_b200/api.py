"""The Python entry point, in the manner of the reference's binding
(bindings/python/quantinfer/__init__.py:36-133): a `Model` opened from a path,
usable as a context manager, with `generate_tokens(tokens, *, max_new_tokens=32,
context_length=None, temperature=0.0, top_k=None, top_p=None,
eos_token_id=EOS_AUTO, seed=0)` returning the generated token ids.

Differences: the path is a model folder (config.json + safetensors) instead of
a converted file; `dtype` selects the bfloat16 or the true 32-bit path; there is
no tokenizer, so `generate`, `tokenize` and `detokenize` raise; and
`generate_batch` runs many prompts through the scheduler at once. Argument
errors raise ValueError, runtime failures QuantInferError, as the reference's
status codes map (bindings/python/quantinfer/_ffi.py:77-84).
"""

from __future__ import annotations

import operator
from threading import RLock

from .errors import QuantInferError
from .sampling import GenerationConfig, Sampler

EOS_AUTO = (1 << 32) - 1


def _unsigned(value, maximum, name):
    value = operator.index(value)
    if not 0 <= value <= maximum:
        raise ValueError(f"{name} is outside its unsigned integer range")
    return value


class Model:
    """A model folder loaded onto one GPU."""

    def __init__(self, path, *, dtype="bfloat16", device="cuda:0", page_size=None, cache_tokens=None,
                 max_requests=8, max_batch_tokens=2048, chunk_size=None, use_graphs=True, run_ahead=True):
        """`run_ahead`: decode steps are launched before the host has read the tokens of the
        step before (engine/pipeline.py); the tokens do not change, they arrive one step late."""
        from .engine import Engine
        from .engine.engine import DEFAULT_PAGE_SIZE

        self._lock = RLock()
        self._engine = Engine.from_folder(
            path, dtype=dtype, device=device, page_size=page_size or DEFAULT_PAGE_SIZE,
            max_tokens=cache_tokens, max_requests=max_requests, use_graphs=use_graphs)
        self._sampler = Sampler.for_engine(self._engine)
        self._max_batch_tokens = max_batch_tokens
        self._chunk_size = chunk_size
        self._run_ahead = run_ahead
        self._open = True

    @classmethod
    def from_engine(cls, engine, *, max_batch_tokens=2048, chunk_size=None, run_ahead=True) -> "Model":
        """A Model over an engine that already exists (random weights made on the device, tests)."""
        self = cls.__new__(cls)
        self._lock = RLock()
        self._engine = engine
        self._sampler = Sampler.for_engine(engine)
        self._max_batch_tokens = max_batch_tokens
        self._chunk_size = chunk_size
        self._run_ahead = run_ahead
        self._open = True
        return self

    # ---- lifetime -------------------------------------------------------------

    def close(self):
        """Release the model once all calls on this handle finish."""
        with self._lock:
            self._engine = None
            self._sampler = None
            self._open = False

    def __enter__(self):
        with self._lock:
            self._require_open()
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        self.close()

    def _require_open(self):
        if not self._open:
            raise QuantInferError("model is closed")

    @property
    def engine(self):
        self._require_open()
        return self._engine

    @property
    def vocab_size(self) -> int:
        return self.engine.spec.vocab_size

    @property
    def max_position_embeddings(self) -> int:
        return self.engine.spec.max_positions

    # ---- no tokenizer ------------------------------------------------------------

    def tokenize(self, text):
        raise QuantInferError("this engine works on token ids; it has no tokenizer")

    def detokenize(self, tokens):
        raise QuantInferError("this engine works on token ids; it has no tokenizer")

    def generate(self, prompt, **options):
        raise QuantInferError("this engine works on token ids; use generate_tokens")

    # ---- generation ----------------------------------------------------------------

    def _config(self, n_prompt, max_new_tokens, context_length, temperature, top_k, top_p, eos_token_id, seed):
        max_new_tokens = _unsigned(max_new_tokens, (1 << 63) - 1, "max_new_tokens")
        if eos_token_id is None:
            eos = None
        else:
            eos_token_id = _unsigned(eos_token_id, EOS_AUTO, "EOS token ID")
            eos = self._engine.spec.eos_token_id if eos_token_id == EOS_AUTO else eos_token_id
        cfg = GenerationConfig(max_new_tokens=max_new_tokens, temperature=float(temperature),
                               top_k=None if top_k is None else _unsigned(top_k, (1 << 63) - 1, "top_k"),
                               top_p=None if top_p is None else float(top_p), eos_token_id=eos,
                               seed=_unsigned(seed, (1 << 64) - 1, "seed"))
        cfg.validate(self._engine.spec.vocab_size)
        context = n_prompt + max_new_tokens if context_length is None else _unsigned(context_length, (1 << 63) - 1, "context_length")
        if context > self._engine.max_seq_len:
            raise ValueError(f"context_length must be between 1 and {self._engine.max_seq_len}")
        if n_prompt + max_new_tokens > context:
            raise ValueError("prompt and max_new_tokens exceed the context length")
        return cfg

    def generate_tokens(self, tokens, *, max_new_tokens=32, context_length=None, temperature=0.0,
                        top_k=None, top_p=None, eos_token_id=EOS_AUTO, seed=0):
        """Generate token IDs. The default uses the model EOS and None disables it."""
        return self.generate_batch([tokens], max_new_tokens=max_new_tokens, context_length=context_length,
                                   temperature=temperature, top_k=top_k, top_p=top_p,
                                   eos_token_id=eos_token_id, seed=seed)[0]

    def generate_batch(self, prompts, *, max_new_tokens=32, context_length=None, temperature=0.0,
                       top_k=None, top_p=None, eos_token_id=EOS_AUTO, seed=0, on_event=None):
        """Generates for every prompt (lists of token ids on the host); returns the
        lists of generated ids in the order of the prompts. Request i draws with
        seed + i."""
        from .engine.pipeline import DecodePipeline
        from .engine.scheduler import FailedEvent, Scheduler, TokenEvent

        with self._lock:
            self._require_open()
            eng = self._engine
            prompts = [[_unsigned(t, EOS_AUTO, "token ID") for t in p] for p in prompts]
            # the sampler reads the step's status word together with the tokens: one wait per step
            sched = Scheduler(eng.cache, lambda entries: eng.step(entries, check_status=False), self._sampler.sample,
                              vocab_size=eng.spec.vocab_size,
                              max_sequences=eng.cache.max_requests,
                              max_tokens=max(self._max_batch_tokens, eng.cache.max_requests),
                              chunk_size=self._chunk_size,
                              pipeline=DecodePipeline(eng, self._sampler) if self._run_ahead and eng.use_graphs else None)
            self.last_scheduler = sched
            ids = []
            for i, p in enumerate(prompts):
                if not p:
                    raise ValueError("a prompt must contain at least one token id")
                cfg = self._config(len(p), max_new_tokens, context_length, temperature, top_k, top_p,
                                   eos_token_id, seed)
                if i:
                    cfg = GenerationConfig(**{**cfg.__dict__, "seed": (cfg.seed + i) % (1 << 64)})
                ids.append(sched.submit(p, cfg))
            out = {rid: [] for rid in ids}
            try:
                for ev in sched.run(on_event):
                    if isinstance(ev, TokenEvent):
                        out[ev.request_id].append(ev.token_id)
                    elif isinstance(ev, FailedEvent):
                        raise QuantInferError(f"request {ev.request_id} failed: {ev.error}")
            finally:
                for rid in list(eng.cache.requests):
                    if rid in out:
                        eng.cache.close(rid)
            return [out[rid] for rid in ids]
