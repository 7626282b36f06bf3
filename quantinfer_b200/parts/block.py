"""Arrangement of a layer's parts: the pre-norm residual block.

    h = h + mixer(norm1(h)) ; h = h + ffn(norm2(h))

The residual stream `resid` is 32-bit; each part's output `delta` is added by
the next norm's fused kernel, so an add never runs alone
(crates/quantinfer-runtime/src/qwen3/mod.rs:117-138: residual :126, norm :127,
attention :128-129, add :130, norm :131-135, feed-forward and add :136-137).
"""

from __future__ import annotations

from .base import Part, build_part, part_class, register_part


class PreNormBlock(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.ffn_norm = build_part("norm", spec.ffn_norm, runtime)
        self.ffn = build_part("ffn", spec.ffn, runtime)
        self._parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    @classmethod
    def needs_of_spec(cls, spec):
        needs = {}
        for cat, sub in (("norm", spec.mixer_norm), ("mixer", spec.mixer),
                         ("norm", spec.ffn_norm), ("ffn", spec.ffn)):
            needs.update(part_class(cat, sub).needs_of_spec(sub))
        return needs

    def load(self, tensors):
        for p in self._parts:
            p.load(tensors)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, resid, delta, batch, cache):
        x = self.mixer_norm(resid, delta)
        a = self.mixer.forward(x, batch, cache)
        x = self.ffn_norm(resid, a)
        return resid, self.ffn.forward(x)


register_part("block", "prenorm", PreNormBlock)
