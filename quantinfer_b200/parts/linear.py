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

    def tensor_core(self, x: torch.Tensor, out_dtype) -> bool:
        return (x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16 and x.shape[0] > 0
                and kernels.gemm_bf16_supported(x.shape[0], self.out_features, self.in_features, out_dtype))

    def forward(self, x: torch.Tensor, out_dtype=None, keep_partials: bool = False) -> torch.Tensor:
        """y = x . W^T. With keep_partials the result may come back as float32 partial sums
        [splits, tokens, out] of a K-split product, for a consumer that adds them itself
        (the fused add + norm does)."""
        out_dtype = out_dtype or x.dtype
        out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
        if x.shape[0] == 0:
            return out
        if self.tensor_core(x, out_dtype):
            return kernels.gemm_bf16(x, self.weight, out, status=self.runtime.status, keep_partials=keep_partials)
        kernels.gemm_simt(x, self.weight, out)
        return out

    def forward_act_mul(self, x: torch.Tensor, activation: str = "silu") -> torch.Tensor:
        """act(gate) * up of a projection whose weight rows are (gate, up) pairs: [tokens, out / 2]. The
        tensor-core product applies silu in its epilogue; any other activation, and any product that is
        not on the tensor cores, writes gate and up and runs the activation kernel over them."""
        half = self.out_features // 2
        act = torch.empty((x.shape[0], half), dtype=x.dtype, device=x.device)
        if x.shape[0] == 0:
            return act
        if activation == "silu" and self.tensor_core(x, x.dtype):
            kernels.gemm_bf16(x, self.weight, act, status=self.runtime.status, epilogue="silu_mul")
            return act
        gu = self.forward(x)
        kernels.act_mul(gu, act, activation, interleaved=True)
        return act

    def forward_silu_mul(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward_act_mul(x, "silu")

    __call__ = forward
