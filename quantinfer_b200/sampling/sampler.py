"""Token selection on the device.

`Sampler.sample(logits, rows)` picks one token per row of float32 logits with
the kernel in csrc/sampling.cu: the first maximum for temperature 0, otherwise
temperature scaling, top-k, top-p and a draw. Each row brings its request's
options and the number of tokens that request has emitted, which is the counter
of its Philox stream; a request's tokens therefore do not depend on what else
is in the batch.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .. import kernels
from .params import GenerationConfig


class Sampler:
    def __init__(self, device, status: torch.Tensor | None = None):
        self.device = torch.device(device)
        self.status = status if status is not None else torch.zeros(1, dtype=torch.int32, device=self.device)

    def sample(self, logits: torch.Tensor, rows: Sequence[tuple]) -> list:
        """`rows[i] = (GenerationConfig, emitted)` for row i of `logits`. Returns token ids."""
        n = logits.shape[0]
        if n != len(rows):
            raise ValueError(f"{n} rows of logits for {len(rows)} requests")
        if n == 0:
            return []
        return self.sample_async(logits, rows).cpu().tolist()

    def sample_async(self, logits: torch.Tensor, rows: Sequence[tuple]) -> torch.Tensor:
        """As `sample`, but returns the device tensor of tokens without waiting."""
        return self.sample_with(logits, self.device_params(rows))

    def sample_with(self, logits: torch.Tensor, params: dict) -> torch.Tensor:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        kernels.sample(logits, params["temperature"], params["top_k"], params["top_p"], params["seed"],
                       params["counter"], out, self.status)
        return out

    def device_params(self, rows: Sequence[tuple]) -> dict:
        """The per-row options as device arrays (None where every row is greedy)."""
        n = len(rows)
        if all(cfg.temperature == 0.0 for cfg, _ in rows):
            return {"temperature": None, "top_k": None, "top_p": None, "seed": None, "counter": None}
        # one int32 block: temperature bits | top_k | top_p bits | counter | seed lo/hi pairs
        buf = np.zeros(6 * n, dtype=np.int32)
        buf[0:n] = np.asarray([cfg.temperature for cfg, _ in rows], dtype=np.float32).view(np.int32)
        buf[n:2 * n] = [min(cfg.top_k, 0x7fffffff) if cfg.top_k else 0 for cfg, _ in rows]
        buf[2 * n:3 * n] = np.asarray([cfg.top_p if cfg.top_p else 0.0 for cfg, _ in rows], dtype=np.float32).view(np.int32)
        buf[3 * n:4 * n] = [emitted for _, emitted in rows]
        buf[4 * n:6 * n] = np.asarray([cfg.seed for cfg, _ in rows], dtype=np.uint64).view(np.int32)
        dev = torch.from_numpy(buf).to(self.device)
        return {"temperature": dev[0:n].view(torch.float32), "top_k": dev[n:2 * n],
                "top_p": dev[2 * n:3 * n].view(torch.float32), "seed": dev[4 * n:6 * n].view(torch.int64),
                "counter": dev[3 * n:4 * n]}
