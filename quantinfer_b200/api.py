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

# The value that stands for "use the model's own end-of-sequence token" in `eos_token_id`; it is the
# largest 32-bit unsigned number, as at the reference's C boundary, so that every real id stays usable.
EOS_AUTO = 0xFFFFFFFF


def _as_count(value, limit: int, what: str) -> int:
    """`value` as a whole number in [0, limit]; anything else is a ValueError naming `what`."""
    n = operator.index(value)
    if n < 0 or n > limit:
        raise ValueError(f"{what} must be a whole number between 0 and {limit}, got {n}")
    return n


class Model:
    """A model folder loaded onto one GPU."""

    def __init__(self, path, *, dtype="bfloat16", device="cuda:0", page_size=None, cache_tokens=None,
                 num_pages=None, max_requests=8, max_batch_tokens=2048, chunk_size=None, use_graphs=True,
                 run_ahead=True, check_finite=False):
        """`run_ahead`: decode steps are launched before the host has read the tokens of the
        step before (engine/pipeline.py); the tokens do not change, they arrive one step late.
        `cache_tokens` or `num_pages` size the page pool; `check_finite` refuses a folder whose
        weights hold NaN or infinities."""
        from .engine import Engine
        from .engine.engine import DEFAULT_PAGE_SIZE

        engine = Engine.from_folder(
            path, dtype=dtype, device=device, page_size=page_size or DEFAULT_PAGE_SIZE, max_tokens=cache_tokens,
            num_pages=num_pages, max_requests=max_requests, use_graphs=use_graphs, check_finite=check_finite)
        self._attach(engine, max_batch_tokens, chunk_size, run_ahead)

    @classmethod
    def from_engine(cls, engine, *, max_batch_tokens=2048, chunk_size=None, run_ahead=True) -> "Model":
        """A Model over an engine that already exists (random weights made on the device, tests)."""
        self = cls.__new__(cls)
        self._attach(engine, max_batch_tokens, chunk_size, run_ahead)
        return self

    def _attach(self, engine, max_batch_tokens, chunk_size, run_ahead) -> None:
        self._lock = RLock()
        self._engine = engine
        self._sampler = Sampler.for_engine(engine)
        self._max_batch_tokens = max_batch_tokens
        self._chunk_size = chunk_size
        self._run_ahead = run_ahead
        self.last_scheduler = None

    # ---- lifetime -------------------------------------------------------------

    def close(self):
        """Drops the engine (weights, cache, graphs). A call that is running on another thread
        holds the lock and ends first; later calls raise."""
        with self._lock:
            self._engine = self._sampler = None

    def __enter__(self):
        self._live()
        return self

    def __exit__(self, *exc_info):
        self.close()
        return False

    def _live(self):
        engine = self._engine
        if engine is None:
            raise QuantInferError("model is closed")
        return engine

    @property
    def engine(self):
        return self._live()

    @property
    def vocab_size(self) -> int:
        return self._live().spec.vocab_size

    @property
    def max_position_embeddings(self) -> int:
        return self._live().spec.max_positions

    # ---- no tokenizer ------------------------------------------------------------

    def tokenize(self, text):
        raise QuantInferError("this engine works on token ids; it has no tokenizer")

    def detokenize(self, tokens):
        raise QuantInferError("this engine works on token ids; it has no tokenizer")

    def generate(self, prompt, **options):
        raise QuantInferError("this engine works on token ids; use generate_tokens")

    # ---- generation ----------------------------------------------------------------

    def _config(self, n_prompt, max_new_tokens, context_length, temperature, top_k, top_p, eos_token_id, seed):
        engine = self._engine
        max_new_tokens = _as_count(max_new_tokens, (1 << 63) - 1, "max_new_tokens")
        eos = None
        if eos_token_id is not None:
            eos = _as_count(eos_token_id, EOS_AUTO, "eos_token_id")
            if eos == EOS_AUTO:
                eos = engine.spec.eos_token_id
        cfg = GenerationConfig(max_new_tokens=max_new_tokens, temperature=float(temperature),
                               top_k=None if top_k is None else _as_count(top_k, (1 << 63) - 1, "top_k"),
                               top_p=None if top_p is None else float(top_p), eos_token_id=eos,
                               seed=_as_count(seed, (1 << 64) - 1, "seed"))
        cfg.validate(engine.spec.vocab_size)
        context = n_prompt + max_new_tokens if context_length is None else _as_count(context_length, (1 << 63) - 1, "context_length")
        if context > engine.max_seq_len:
            raise ValueError(f"context_length must be between 1 and {engine.max_seq_len}")
        if n_prompt + max_new_tokens > context:
            raise ValueError("prompt and max_new_tokens exceed the context length")
        return cfg

    def generate_tokens(self, tokens, *, max_new_tokens=32, context_length=None, temperature=0.0,
                        top_k=None, top_p=None, eos_token_id=EOS_AUTO, seed=0):
        """The ids generated after the prompt `tokens` (a list of ids on the host). `eos_token_id`:
        EOS_AUTO stops at the end-of-sequence id that config.json names (if it names one), an id
        stops at that id, None never stops early; the stopping token is part of the result."""
        return self.generate_batch([tokens], max_new_tokens=max_new_tokens, context_length=context_length,
                                   temperature=temperature, top_k=top_k, top_p=top_p,
                                   eos_token_id=eos_token_id, seed=seed)[0]

    def generate_batch(self, prompts, *, max_new_tokens=32, context_length=None, temperature=0.0,
                       top_k=None, top_p=None, eos_token_id=EOS_AUTO, seed=0, on_event=None):
        """Generates for every prompt (lists of token ids on the host); returns the
        lists of generated ids in the order of the prompts. Request i draws with
        seed + i."""
        from .engine.generation import run_requests

        with self._lock:
            engine = self._live()
            prompts = [[_as_count(t, EOS_AUTO, "token id") for t in p] for p in prompts]
            configs = []
            for i, p in enumerate(prompts):
                if not p:
                    raise ValueError("a prompt must contain at least one token id")
                cfg = self._config(len(p), max_new_tokens, context_length, temperature, top_k, top_p,
                                   eos_token_id, seed)
                if i:
                    cfg = GenerationConfig(**{**cfg.__dict__, "seed": (cfg.seed + i) % (1 << 64)})
                configs.append(cfg)
            run = run_requests(engine, self._sampler, prompts, configs, max_batch_tokens=self._max_batch_tokens,
                               chunk_size=self._chunk_size, run_ahead=self._run_ahead, on_event=on_event)
            self.last_scheduler = run.scheduler
            self.last_run = run
            return [r.tokens for r in run.results]
