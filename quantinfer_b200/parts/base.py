"""What every part is, and the registry that builds parts from their specs.

A part is built from its spec and a :class:`Runtime` and knows nothing of the
model it sits in. The interfaces:

* every part: `tensor_needs() -> {file name: TensorNeed}` and
  `load({file name: CPU tensor})`;
* norm: `forward(resid, delta, rows=None, write_resid=True) -> normed`
  (fused `resid += delta`, then the norm; `rows` gathers source rows);
* position encoding: whatever its mixers ask of it (the rotary part offers
  `cos`, `sin`, `rotary_dim`);
* mixer: `cache_need() -> PagedKVNeed | StateNeed | None` and
  `forward(x, batch, cache) -> y`, x and y `[tokens, hidden]` in the activation
  type, `batch` a :class:`StepBatch`, `cache` the :class:`CacheView` of the
  layer call;
* feed-forward: `forward(x) -> y`;
* block: `forward(resid, delta, batch, cache) -> (resid, delta)`: the 32-bit
  residual stream and the not-yet-added output of the last part.

Kinds are registered per category with :func:`register_part`; a spec's `kind`
selects the class, so a new part needs no change to existing files.

What a mixer reads of the step. The batch's device arrays are its interface:
`q_start[i] .. q_start[i + 1]` are entry i's rows of `x`, `start_pos[i]` the
position of its first token, `kv_len[i]` its context after the step,
`slot_ids[i]` its slot (the row of a `StateNeed` tensor), `token_req[t]` and
`positions[t]` the entry and position of row t, `block_tables[cache.group]`
its pages. Decode steps are replayed from CUDA graphs and launched before the
host has read the step before, so a mixer must work from these arrays alone,
with kernels or torch operations whose shapes depend only on the batch's counts
(`n_tokens`, `n_requests`); the batch's host-side lists raise in such a step.
State of fixed size is saved by the cache manager before a step and restored
if the step fails; a mixer only reads and writes `cache.state[slot]`.

Partial sums. A projection whose product was cut along K may hand back the
32-bit partial sums `[splits, tokens, width]` instead of their sum, when asked
to (`Linear.forward(keep_partials=True)`); a part does that only for its own
output `delta`, which the block passes to the next norm. So a norm's `delta` is
either `[tokens, hidden]` in the activation type or `[splits, tokens, hidden]`
in float32, to be added in split order; `parts.norm.sum_partials` turns the
second into the first for a norm that has no kernel for it. A part that never
asks for partial sums never sees any.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..errors import ConfigError

CATEGORIES = ("norm", "position", "mixer", "ffn", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, type]] = {c: {} for c in CATEGORIES}


@dataclass
class Runtime:
    """What parts share: the activation type, the device, the device status word
    that kernels set bits in instead of trapping, and a place to share built
    tables (rotary tables are the same for every layer)."""

    dtype: torch.dtype
    device: torch.device
    status: torch.Tensor = None
    shared: dict = field(default_factory=dict)
    io: torch.Tensor = None      # int32: [0] is the status word, the rest takes sampled tokens (one D2H reads both)

    def __post_init__(self):
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ConfigError(f"the activation type must be float32 or bfloat16, got {self.dtype}")
        self.device = torch.device(self.device)
        if self.status is None:
            self.io = torch.zeros(1 + 8192, dtype=torch.int32, device=self.device)
            self.status = self.io[0:1]


def register_part(category: str, kind: str, cls: type) -> None:
    if category not in _REGISTRY:
        raise ConfigError(f"unknown part category {category!r}; one of {CATEGORIES}")
    _REGISTRY[category][kind] = cls


def part_class(category: str, spec) -> type:
    kind = getattr(spec, "kind", None)
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        raise ConfigError(
            f"no {category} part of kind {kind!r} is registered (known: {sorted(_REGISTRY.get(category, {}))})") from None


def build_part(category: str, spec, runtime: Runtime):
    return part_class(category, spec)(spec, runtime)


class Part:
    """Base of all parts: no tensors unless a subclass says so."""

    def __init__(self, spec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime

    @classmethod
    def needs_of_spec(cls, spec) -> dict:
        """{file name: TensorNeed} of a part with this spec; needs no device."""
        return {}

    def tensor_needs(self) -> dict:
        return type(self).needs_of_spec(self.spec)

    def device_tensors(self) -> list:
        """Every tensor this part and its sub-parts hold on the device."""
        out = []
        for v in vars(self).values():
            items = v if isinstance(v, (list, tuple)) else (v,)
            for x in items:
                if isinstance(x, torch.Tensor):
                    out.append(x)
                elif isinstance(x, Part):
                    out += x.device_tensors()
                elif hasattr(x, "weight") and isinstance(getattr(x, "weight"), torch.Tensor):
                    out.append(x.weight)
        return out

    def load(self, tensors: dict) -> None:
        pass

    def _gain(self, t: torch.Tensor) -> torch.Tensor:
        """Norm gains are used in 32-bit whatever they were stored as."""
        return t.to(device=self.runtime.device, dtype=torch.float32).contiguous()
