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
from ..errors import QuantInferError


class Sampler:
    def __init__(self, device, status: torch.Tensor | None = None, io: torch.Tensor | None = None):
        """`io` (int32, [0] the status word, then room for tokens) lets `sample` read the
        tokens and the status of the step that produced the logits in one transfer."""
        self.device = torch.device(device)
        self.io = io
        if io is not None:
            self.status = io[0:1]
        else:
            self.status = status if status is not None else torch.zeros(1, dtype=torch.int32, device=self.device)
        self._pinned = [None] * 4        # staging for the per-row options, used in turn
        self._pinned_event = [None] * 4
        self._turn = 0

    @classmethod
    def for_engine(cls, engine) -> "Sampler":
        self = cls(engine.device, io=engine.runtime.io)
        self.engine = engine
        return self

    def sample_step(self, logits: torch.Tensor, rows: Sequence[tuple]) -> list:
        """As `sample`, for the logits of the engine's last step and requests whose slot records were
        written (`Engine.assign_sampling`): the kernel reads each row's options from its request's record,
        found through the step's device arrays, and advances the record's counter; nothing is uploaded.
        `rows` only says how many rows there are and whether any of them draws."""
        n = logits.shape[0]
        if n != len(rows):
            raise ValueError(f"{n} rows of logits for {len(rows)} requests")
        if n == 0:
            return []
        engine = getattr(self, "engine", None)
        batch = engine.last_batch if engine is not None else None
        if batch is None or self.io is None or n + 1 > self.io.numel() or batch.n_logit_rows != n:
            return self.sample(logits, rows)
        out = self.io[1:1 + n]
        greedy = all(cfg.temperature == 0.0 for cfg, _ in rows)
        kernels.sample_slots(logits, batch.logit_rows, batch.token_req, batch.slot_ids, engine.slots.table, greedy,
                             out, self.status)
        host = self.io[:1 + n].cpu().tolist()          # waits for the step; status and tokens together
        if host[0]:
            self.status.zero_()
            raise QuantInferError(f"the step failed on the device (status {host[0]}: "
                                  + "; ".join(kernels.status_names(host[0])) + ")")
        return host[1:]

    def sample(self, logits: torch.Tensor, rows: Sequence[tuple]) -> list:
        """`rows[i] = (GenerationConfig, emitted)` for row i of `logits`. Returns token ids."""
        n = logits.shape[0]
        if n != len(rows):
            raise ValueError(f"{n} rows of logits for {len(rows)} requests")
        if n == 0:
            return []
        params = self.device_params(rows)
        if self.io is None or n + 1 > self.io.numel():
            return self.sample_with(logits, params).cpu().tolist()
        out = self.io[1:1 + n]
        kernels.sample(logits, params["temperature"], params["top_k"], params["top_p"], params["seed"],
                       params["counter"], out, self.status)
        host = self.io[:1 + n].cpu().tolist()          # waits for the step; status and tokens together
        if host[0]:
            self.status.zero_()
            raise QuantInferError(f"the step failed on the device (status {host[0]}: "
                                  + "; ".join(kernels.status_names(host[0])) + ")")
        return host[1:]

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
        dev = self._to_device(buf)
        return {"temperature": dev[0:n].view(torch.float32), "top_k": dev[n:2 * n],
                "top_p": dev[2 * n:3 * n].view(torch.float32), "seed": dev[4 * n:6 * n].view(torch.int64),
                "counter": dev[3 * n:4 * n]}

    def _to_device(self, buf: np.ndarray) -> torch.Tensor:
        """Copies through pinned memory without waiting for the stream (steps may run ahead of the host)."""
        turn = self._turn
        self._turn = (turn + 1) % len(self._pinned)
        host = self._pinned[turn]
        if host is None or host.numel() < buf.size:
            host = self._pinned[turn] = torch.empty(max(2 * buf.size, 256), dtype=torch.int32, pin_memory=True)
            self._pinned_event[turn] = torch.cuda.Event()
        else:
            self._pinned_event[turn].synchronize()      # the copy that last used this buffer is done
        host[:buf.size].numpy()[:] = buf
        dev = host[:buf.size].to(self.device, non_blocking=True)
        self._pinned_event[turn].record()
        return dev
