"""RMSNorm with the residual add fused in.

    x = resid + delta ; resid = x ; out = (x / sqrt(mean(x^2) + eps)) * gain

The gain multiplies as stored (no `1 + g`), and one eps serves every norm of
the model, as in the reference (backends/cpu/src/backend.rs:172-193; placement
crates/quantinfer-runtime/src/qwen3/mod.rs:127,131-135,370-372). Sums are 32-bit.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorNeed
from .base import Part, register_part


def sum_partials(delta, dtype=None):
    """`delta` as one [tokens, hidden] tensor: the K-split partial sums [splits, tokens, hidden]
    of a projection added in split order (32-bit), or `delta` itself when it is already whole.
    For norms that have no kernel that adds the partial sums itself."""
    if delta is None or delta.dim() == 2:
        return delta
    total = delta[0].clone()
    for k in range(1, delta.shape[0]):
        total += delta[k]
    return total if dtype is None else total.to(dtype)


class RMSNorm(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.gain = None

    @classmethod
    def needs_of_spec(cls, spec):
        return {spec.prefix + "weight": TensorNeed((spec.size,), "gain", "gain")}

    def load(self, tensors):
        self.gain = self._gain(tensors[self.spec.prefix + "weight"])

    def forward(self, resid, delta, rows=None, write_resid=True):
        n = resid.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=self.runtime.dtype, device=resid.device)
        kernels.add_rmsnorm(resid, delta, self.gain, self.spec.eps, out, rows=rows, write_resid=write_resid)
        return out

    __call__ = forward


register_part("norm", "rmsnorm", RMSNorm)
