"""Rotary position encoding.

For pair p < rotary_dim / 2 of a head: angle = position * theta^(-2p / rotary_dim),
all in 32-bit; the pair's two elements are rotated by it
(crates/quantinfer-runtime/src/attention.rs:7-36, the angle :29-32;
backends/cpu/src/backend.rs:240-280, the rotation :270-275). Which two elements
form pair p is the spec's `pairing`: "half_split" (x[p], x[p + rotary_dim/2]),
the reference's rule for this architecture, or "interleaved" (x[2p], x[2p + 1]),
the order its converter writes for others
(crates/quantinfer-format/src/gguf/layout.rs:52-55). The part owns the table
and the rule: inverse frequencies are computed once in 32-bit, the cos/sin
table [max_positions, rotary_dim / 2] is built on the device, and the mixer's
kernel looks positions up in it and pairs as `pairing` says. Tables are shared
between layers with the same angles.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..errors import ConfigError
from .base import Part, register_part


class RopeHalfSplit(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ConfigError(f"rotary_dim {spec.rotary_dim} must be even and within head_dim {spec.head_dim}")
        self.rotary_dim = spec.rotary_dim
        self.pairing = getattr(spec, "pairing", "half_split")
        if self.pairing not in ("half_split", "interleaved"):
            raise ConfigError(f"rotary pairing {self.pairing!r} is not known (half_split or interleaved)")
        key = ("rope_half_split", spec.rotary_dim, float(spec.theta), spec.max_positions)
        if key not in runtime.shared:
            half = spec.rotary_dim // 2
            # exponent = 2p / rotary_dim and theta^(-exponent), both in 32-bit
            exponent = (2.0 * torch.arange(half, dtype=torch.float32)) / torch.tensor(float(spec.rotary_dim), dtype=torch.float32)
            inv_freq = torch.pow(torch.tensor(spec.theta, dtype=torch.float32), -exponent)
            runtime.shared[key] = kernels.rope_table(inv_freq.to(runtime.device), spec.max_positions)
        self.cos, self.sin = runtime.shared[key]
        self.max_positions = spec.max_positions


register_part("position", "rope_half_split", RopeHalfSplit)
