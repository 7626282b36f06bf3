"""Descriptions of a model as data: parts with their sizes and constants, the
layers they form, and the order in which layers run.

An architecture's config class turns its config.json into a :class:`ModelSpec`.
Nothing below the spec knows which architecture it came from: parts are built
from their spec alone (`parts.registry.build_*`). The reference keeps the same
split between a config and an architecture-neutral description
(crates/quantinfer-model/src/semantic.rs:39-57,91-103: per-layer attention,
normalisation, activation and positional specs).

Each spec carries `kind`, the key under which the part's class is registered,
and `prefix`, prepended to the part's local tensor names to give the names in
the weight files.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    prefix: str = ""
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class PositionSpec:
    """Rotary encoding over the first `rotary_dim` dimensions of each head, angle of pair p =
    position * theta^(-2p / rotary_dim). `pairing` says which two elements pair p is:
    "half_split" (p, p + rotary_dim / 2) or "interleaved" (2p, 2p + 1)."""

    head_dim: int
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope_half_split"
    pairing: str = "half_split"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged key/value cache."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: Optional[PositionSpec]
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    window: Optional[int] = None      # None: all earlier keys; n: the last n keys
    scale: Optional[float] = None     # None: head_dim ** -0.5
    prefix: str = ""
    kind: str = "attention"


@dataclass(frozen=True)
class FeedForwardSpec:
    """Gated feed-forward: down(act(gate(x)) * up(x))."""

    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    prefix: str = ""
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class LayerSpec:
    """One block: x += mixer(norm(x)); x += ffn(norm(x)) for kind `prenorm`."""

    mixer_norm: NormSpec
    mixer: object          # a mixer spec (AttentionSpec or any registered kind)
    ffn_norm: NormSpec
    ffn: object            # a feed-forward spec
    kind: str = "prenorm"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run `layer` with cache entry `cache`.

    Naming a layer twice reuses its weights. `writes_cache=False` makes the
    call read a cache entry that an earlier call filled, without adding to it.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int
    prefix: str = ""
    kind: str = "embedding"


@dataclass(frozen=True)
class HeadSpec:
    vocab_size: int
    hidden_size: int
    tied: bool              # True: the head is the embedding table
    prefix: str = ""
    kind: str = "lm_head"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: tuple
    order: tuple
    final_norm: NormSpec
    head: HeadSpec
    eos_token_id: Optional[int] = None
    extra: dict = field(default_factory=dict, compare=False)

    def cache_entries(self) -> int:
        return 1 + max(call.cache for call in self.order) if self.order else 0

    def validate(self) -> None:
        from ..errors import ConfigError

        if not self.layers or not self.order:
            raise ConfigError("a model needs at least one layer and one entry in its run order")
        written = set()
        for i, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ConfigError(f"run order entry {i} names layer {call.layer}, the model has {len(self.layers)}")
            if call.cache < 0:
                raise ConfigError(f"run order entry {i} has a negative cache entry")
            if call.writes_cache:
                if call.cache in written:
                    raise ConfigError(f"run order entry {i}: cache entry {call.cache} already has a writer")
                written.add(call.cache)
            elif call.cache not in written:
                raise ConfigError(f"run order entry {i} reads cache entry {call.cache} before any layer wrote it")
        if written != set(range(self.cache_entries())):
            raise ConfigError("cache entries must be numbered 0..n-1 and each needs a writer")
