"""Token embedding (a row gather into the 32-bit residual stream) and the
output head (a projection of the normed rows to 32-bit logits).

A tied head uses the embedding table itself: [vocab, hidden] is already the
[out, in] layout the projection reads (the reference materialises a transposed
copy, crates/quantinfer-runtime/src/qwen3/loader.rs:59; the gather is
backends/cpu/src/backend.rs:282-298, the head crates/quantinfer-runtime/src/qwen3/mod.rs:369-378).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear


class Embedding(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.table = Linear(runtime, spec.vocab_size, spec.hidden_size, spec.prefix + "weight")

    @classmethod
    def needs_of_spec(cls, spec):
        return {spec.prefix + "weight": TensorNeed((spec.vocab_size, spec.hidden_size), "table")}

    def load(self, tensors):
        self.table.load(tensors[self.spec.prefix + "weight"])

    def forward(self, token_ids):
        out = torch.empty((token_ids.numel(), self.spec.hidden_size), dtype=torch.float32, device=token_ids.device)
        kernels.embedding(self.table.weight, token_ids, out, self.runtime.status)
        return out

    __call__ = forward


class LMHead(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.proj = None if spec.tied else Linear(runtime, spec.vocab_size, spec.hidden_size, spec.prefix + "weight")

    @classmethod
    def needs_of_spec(cls, spec):
        if spec.tied:
            return {}
        return {spec.prefix + "weight": TensorNeed((spec.vocab_size, spec.hidden_size))}

    def load(self, tensors):
        if not self.spec.tied:
            self.proj.load(tensors[self.spec.prefix + "weight"])

    def tie(self, embedding: Embedding):
        self.proj = embedding.table

    def forward(self, x):
        return self.proj(x, out_dtype=torch.float32)

    __call__ = forward


register_part("embedding", "embedding", Embedding)
register_part("head", "lm_head", LMHead)
