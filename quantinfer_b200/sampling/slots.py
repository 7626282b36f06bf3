"""The per-request slot's sampling record, kept on the device.

A request that the cache manager has opened owns a slot, an index into arrays
of fixed size. What the sampler needs of a request lives in one such array, a
record of eight 32-bit words per slot on the device:

    word 0  temperature (float bits)      word 4, 5  seed, low and high word
    word 1  top_k (0: none)               word 6     max_new_tokens
    word 2  top_p (float bits, 0: none)   word 7     eos token id (-1: none)
    word 3  tokens emitted so far: the counter of the request's random stream

The host writes a record once, when the request is admitted (`assign`, one copy
of 32 bytes in stream order); from then on the sampling kernel reads the options
by slot, found through the step's own device arrays, and advances the count of
emitted tokens itself. A step therefore uploads nothing for the sampler, and a
decode step that runs ahead of the host draws with the right counter without the
host telling it. The rest of what a request keeps per slot, its position and its
block tables, belongs to the cache manager: the host decides them anew for every
step and they travel with the step's batch arrays.

The reference keeps the same things in its session (configuration, tokens
emitted, next input: crates/quantinfer-runtime/src/session.rs:64-70) and draws
from a hash of the logits that never advances (generation.rs:219-230); the
record and the counter-based stream are this engine's.
"""

from __future__ import annotations

import numpy as np
import torch

from .params import GenerationConfig

SLOT_WORDS = 8


class RequestSlots:
    def __init__(self, num_slots: int, device):
        self.num_slots = num_slots
        self.device = torch.device(device)
        self.table = torch.zeros((num_slots, SLOT_WORDS), dtype=torch.int32, device=self.device)
        self._pinned = torch.zeros((num_slots, SLOT_WORDS), dtype=torch.int32, pin_memory=True)
        self._host = self._pinned.numpy()
        self.configs = [None] * num_slots          # what was assigned, for the host's own decisions

    def assign(self, slot: int, config: GenerationConfig, emitted: int = 0) -> None:
        """Writes the record of `slot`: the request's options and how many tokens it has emitted
        (not zero for a request that is taken up again after a preemption)."""
        if not 0 <= slot < self.num_slots:
            raise ValueError(f"slot {slot} is outside the {self.num_slots} slots")
        row = self._host[slot]
        row[0] = np.float32(config.temperature).view(np.int32)
        row[1] = min(config.top_k, 0x7FFFFFFF) if config.top_k else 0
        row[2] = np.float32(config.top_p if config.top_p else 0.0).view(np.int32)
        row[3] = emitted
        row[4:6] = np.asarray([config.seed], dtype=np.uint64).view(np.int32)
        row[6] = min(config.max_new_tokens, 0x7FFFFFFF)
        row[7] = -1 if config.eos_token_id is None else config.eos_token_id
        self.table[slot].copy_(self._pinned[slot], non_blocking=True)
        self.configs[slot] = config

    def all_greedy(self, slots) -> bool:
        return all(self.configs[s] is not None and self.configs[s].temperature == 0.0 for s in slots)
