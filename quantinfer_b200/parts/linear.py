"""A bias-free projection y = x . W^T with W in the checkpoint's [out, in] layout.

Which kernel runs is decided here, once per call, from the element types:

* activation type float32: the 32-bit FMA product (true 32-bit path, no tensor cores);
* bfloat16 activations and bfloat16 weights: the tcgen05 tensor-core product
  (32-bit accumulation), when its constraints hold (K a multiple of 8 for the
  16-byte rule of TMA, see `kernels.gemm_bf16_supported`);
* anything else (a weight stored in 32-bit under bfloat16 activations, odd K):
  the 32-bit FMA product with mixed operand types.

The reference has one projection type per storage format and no bias field
(crates/quantinfer-runtime/src/linear.rs:14-30,57-74).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..errors import WeightError


class Linear:
    def __init__(self, runtime, out_features: int, in_features: int, name: str = "linear"):
        self.runtime = runtime
        self.out_features = out_features
        self.in_features = in_features
        self.name = name
        self.weight = None

    def load(self, w: torch.Tensor) -> None:
        if tuple(w.shape) != (self.out_features, self.in_features):
            raise WeightError(f"{self.name}: weight has shape {list(w.shape)}, expected {[self.out_features, self.in_features]}")
        rt = self.runtime
        if rt.dtype == torch.float32:
            w = w.to(device=rt.device, dtype=torch.float32)
        else:
            w = w.to(device=rt.device)  # bfloat16 stays bfloat16, a 32-bit tensor stays 32-bit
        self.weight = w.contiguous()

    def forward(self, x: torch.Tensor, out_dtype=None, out=None) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        if out is None:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
        if x.shape[0] == 0:
            return out
        if (x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16
                and kernels.gemm_bf16_supported(x.shape[0], self.out_features, self.in_features, out.dtype)):
            kernels.gemm_bf16(x, self.weight, out)
        else:
            kernels.gemm_simt(x, self.weight, out)
        return out

    __call__ = forward
