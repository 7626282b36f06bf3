"""Gated feed-forward: y = down(act(gate(x)) * up(x)), no biases; act is the spec's `activation`
(silu for this architecture: SwiGLU; gelu, gelu_tanh and relu have kernels too).

gate and up are interleaved row by row into one [2I, H] weight at load (row 2i
gate, row 2i + 1 up), so that one product computes both and the thread that
holds a (gate, up) pair applies the activation in the product's epilogue. The reference runs them as two products followed
by silu(g) * u in the division form and the down projection
(crates/quantinfer-runtime/src/qwen3/mod.rs:194-209; backends/cpu/src/backend.rs:224-238).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear


class GatedMLP(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.activation not in kernels.ACTIVATIONS:
            raise ConfigError(f"gated_mlp: activation {spec.activation!r} has no kernel (one of {sorted(kernels.ACTIVATIONS)})")
        h, i = spec.hidden_size, spec.intermediate_size
        self.gate_up = Linear(runtime, 2 * i, h, spec.prefix + "gate_up_proj")
        self.down = Linear(runtime, h, i, spec.prefix + "down_proj")

    @classmethod
    def needs_of_spec(cls, spec):
        h, i, p = spec.hidden_size, spec.intermediate_size, spec.prefix
        return {
            p + "gate_proj.weight": TensorNeed((i, h)),
            p + "up_proj.weight": TensorNeed((i, h)),
            p + "down_proj.weight": TensorNeed((h, i)),
        }

    def load(self, tensors):
        p = self.spec.prefix
        g, u = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        self.gate_up.load(torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1]))
        self.down.load(tensors[p + "down_proj.weight"])

    def forward(self, x):
        return self.down(self.gate_up.forward_act_mul(x, self.spec.activation), keep_partials=True)

    __call__ = forward


register_part("ffn", "gated_mlp", GatedMLP)
