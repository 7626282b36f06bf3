"""Options of generation and their checks.

Names, defaults and validation are the reference's `GenerationConfig`
(crates/quantinfer-runtime/src/generation.rs:8-55): max_new_tokens 128 and > 0,
temperature 0 (greedy) and finite >= 0, top_k absent or > 0, top_p absent or in
(0, 1], eos_token_id absent or inside the vocabulary, seed a 64-bit unsigned.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class GenerationConfig:
    max_new_tokens: int = 128
    temperature: float = 0.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    eos_token_id: Optional[int] = None
    seed: int = 0

    def validate(self, vocab_size: Optional[int] = None) -> None:
        if isinstance(self.max_new_tokens, bool) or not isinstance(self.max_new_tokens, int) or self.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be greater than zero")
        if not isinstance(self.temperature, (int, float)) or not math.isfinite(self.temperature) or self.temperature < 0.0:
            raise ValueError("temperature must be finite and non-negative")
        if self.top_k is not None and (isinstance(self.top_k, bool) or not isinstance(self.top_k, int) or self.top_k <= 0):
            raise ValueError("top_k must be greater than zero when provided")
        if self.top_p is not None and (not math.isfinite(self.top_p) or not 0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be finite and in the range (0, 1]")
        if not isinstance(self.seed, int) or not 0 <= self.seed < (1 << 64):
            raise ValueError("seed must be an unsigned 64-bit integer")
        if self.eos_token_id is not None:
            if isinstance(self.eos_token_id, bool) or not isinstance(self.eos_token_id, int) or self.eos_token_id < 0:
                raise ValueError("eos_token_id must be a non-negative integer")
            if vocab_size is not None and self.eos_token_id >= vocab_size:
                raise ValueError("EOS token id is outside the model vocabulary")
