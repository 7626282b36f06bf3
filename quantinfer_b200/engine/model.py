"""The model, assembled from a :class:`ModelSpec`: embedding, blocks run in the
spec's order, final norm on the wanted rows, head.

Nothing here is specific to an architecture; the spec says which parts there
are. The forward pass is the reference's `forward_hidden` and `project_logits`
(crates/quantinfer-runtime/src/qwen3/mod.rs:345-378) with its
`last_hidden_rows` gather before the final norm (batch.rs:247-289;
mod.rs:339-342), generalised to any wanted rows.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import ModelSpec
from ..errors import ConfigError
from ..parts import Runtime, build_part, part_class


def tensor_needs_of_spec(spec: ModelSpec) -> dict:
    """{file name: TensorNeed} of the whole model, in a fixed order; needs no device."""
    needs = {}
    needs.update(part_class("embedding", spec.embedding).needs_of_spec(spec.embedding))
    for layer in spec.layers:
        needs.update(part_class("block", layer).needs_of_spec(layer))
    needs.update(part_class("norm", spec.final_norm).needs_of_spec(spec.final_norm))
    needs.update(part_class("head", spec.head).needs_of_spec(spec.head))
    return needs


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.blocks = [build_part("block", layer, runtime) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.head = build_part("head", spec.head, runtime)
        if spec.head.tied:
            self.head.tie(self.embedding)
        self.order = spec.order
        self.native = None            # the C++ driver's description of this model (engine/native.py), once asked for
        self.use_native = True
        # what each cache entry must hold comes from the layer that writes it
        self.cache_needs = [None] * spec.cache_entries()
        for call in self.order:
            if call.writes_cache:
                self.cache_needs[call.cache] = self.blocks[call.layer].cache_need()
        for call in self.order:
            if not call.writes_cache and self.blocks[call.layer].cache_need() != self.cache_needs[call.cache]:
                raise ConfigError(
                    f"layer {call.layer} reads cache entry {call.cache}, whose writer keeps something else")

    def _parts(self):
        return (self.embedding, *self.blocks, self.final_norm, self.head)

    def tensor_needs(self) -> dict:
        needs = {}
        for part in self._parts():
            needs.update(part.tensor_needs())
        return needs

    def load(self, tensors: dict) -> None:
        for part in self._parts():
            part.load(tensors)

    def weight_bytes(self) -> int:
        """Bytes of distinct device tensors the parts hold (a tied head counts once)."""
        seen, total = set(), 0
        for part in self._parts():
            for t in part.device_tensors():
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    def forward(self, batch, cache_views) -> torch.Tensor:
        """Runs the batch's tokens; returns float32 logits [len(batch.logit_rows), vocab]. A model whose
        parts are all of the kinds the library's C++ driver knows runs through it (one call a step);
        any other, and any step while kernels are being left out for a measurement, runs part by part."""
        if self.use_native and not kernels.knock_out:
            if self.native is None:
                from .native import NativeProgram

                self.native = NativeProgram.build(self, cache_views) or False
            if self.native:
                return self.native.forward(batch)
        resid = self.embedding(batch.token_ids)
        delta = None
        for call, view in zip(self.order, cache_views):
            resid, delta = self.blocks[call.layer].forward(resid, delta, batch, view)
        if batch.n_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=resid.device)
        normed = self.final_norm(resid, delta, rows=batch.logit_rows)
        return self.head(normed)
