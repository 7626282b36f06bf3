"""Typed configuration of Qwen3 dense (`Qwen3ForCausalLM`), read from the keys
of its config.json.

Keys, defaults and checks follow the reference's `Qwen3Config`
(crates/quantinfer-model/src/qwen3.rs:11-37 fields, :39-45 defaults, :52-55
effective head size, :57-119 validation, :121-131 derived sizes). Unknown keys
are ignored, as there (no `deny_unknown_fields`). Every size and constant of
the model comes from here; none stands in the code of the parts.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional

from ..errors import ConfigError
from .spec import (AttentionSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerCall, LayerSpec,
                   ModelSpec, NormSpec, PositionSpec)

ARCHITECTURE = "Qwen3ForCausalLM"

# Defaults of absent keys (crates/quantinfer-model/src/qwen3.rs:39-45).
_DEFAULT_RMS_NORM_EPS = 1e-6
_DEFAULT_ROPE_THETA = 1_000_000.0

_REQUIRED_INTS = (
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
)


def _int(d: dict, key: str, required: bool) -> Optional[int]:
    if key not in d or d[key] is None:
        if required:
            raise ConfigError(f"config.json has no `{key}`")
        return None
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json `{key}` must be an integer, got {v!r}")
    if v < 0:
        raise ConfigError(f"config.json `{key}` must not be negative, got {v}")
    return v


def _float(d: dict, key: str, default: float) -> float:
    if key not in d or d[key] is None:
        return default
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json `{key}` must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    max_position_embeddings: int
    head_dim: Optional[int] = None
    rms_norm_eps: float = _DEFAULT_RMS_NORM_EPS
    rope_theta: float = _DEFAULT_ROPE_THETA
    tie_word_embeddings: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    use_sliding_window: bool = False
    rope_scaling: Any = None
    architectures: tuple = ()
    model_type: Optional[str] = None
    eos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = field(default=None, compare=False)

    # ---- reading -----------------------------------------------------

    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        if not isinstance(d, dict):
            raise ConfigError("config.json must hold a JSON object")
        ints = {k: _int(d, k, True) for k in _REQUIRED_INTS}
        tie = d.get("tie_word_embeddings", False)
        usw = d.get("use_sliding_window", False)
        for key, v in (("tie_word_embeddings", tie), ("use_sliding_window", usw)):
            if not isinstance(v, bool):
                raise ConfigError(f"config.json `{key}` must be true or false, got {v!r}")
        arch = d.get("architectures") or []
        if not isinstance(arch, list) or any(not isinstance(a, str) for a in arch):
            raise ConfigError("config.json `architectures` must be a list of strings")
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        if eos is not None and (isinstance(eos, bool) or not isinstance(eos, int)):
            raise ConfigError(f"config.json `eos_token_id` must be an integer, got {eos!r}")
        cfg = cls(
            **ints,
            head_dim=_int(d, "head_dim", False),
            rms_norm_eps=_float(d, "rms_norm_eps", _DEFAULT_RMS_NORM_EPS),
            rope_theta=_float(d, "rope_theta", _DEFAULT_ROPE_THETA),
            tie_word_embeddings=tie,
            sliding_window=_int(d, "sliding_window", False),
            max_window_layers=_int(d, "max_window_layers", False),
            use_sliding_window=usw,
            rope_scaling=d.get("rope_scaling"),
            architectures=tuple(arch),
            model_type=d.get("model_type"),
            eos_token_id=eos,
            torch_dtype=d.get("torch_dtype") or d.get("dtype"),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, text: str) -> "Qwen3Config":
        try:
            d = json.loads(text)
        except json.JSONDecodeError as exc:
            raise ConfigError(f"config.json is not valid JSON: {exc}") from exc
        return cls.from_dict(d)

    @classmethod
    def from_folder(cls, folder) -> "Qwen3Config":
        path = Path(folder) / "config.json"
        if not path.is_file():
            raise ConfigError(f"{path} does not exist")
        return cls.from_json(path.read_text())

    def to_dict(self) -> dict:
        d = {
            "architectures": list(self.architectures) or [ARCHITECTURE],
            "model_type": self.model_type or "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.effective_head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
        }
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        if self.torch_dtype:
            d["torch_dtype"] = self.torch_dtype
        return d

    # ---- derived sizes ----------------------------------------------

    @property
    def effective_head_dim(self) -> int:
        if self.head_dim is not None:
            return self.head_dim
        return self.hidden_size // max(self.num_attention_heads, 1)

    @property
    def query_projection_size(self) -> int:
        return self.num_attention_heads * self.effective_head_dim

    @property
    def key_value_projection_size(self) -> int:
        return self.num_key_value_heads * self.effective_head_dim

    @property
    def kv_group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # ---- checks ------------------------------------------------------

    def validate(self) -> None:
        for key in _REQUIRED_INTS:
            if getattr(self, key) <= 0:
                raise ConfigError(f"Qwen3 `{key}` must be greater than zero")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"attention heads ({self.num_attention_heads}) must be divisible by key/value heads "
                f"({self.num_key_value_heads})")
        if self.head_dim is not None and self.head_dim == 0:
            raise ConfigError("head_dim must be greater than zero")
        if self.head_dim is None and self.hidden_size % self.num_attention_heads:
            raise ConfigError("hidden size must be divisible by attention heads when head_dim is absent")
        if self.effective_head_dim % 2:
            raise ConfigError("head_dim must be even for RoPE")
        for key in ("rms_norm_eps", "rope_theta"):
            v = getattr(self, key)
            if not math.isfinite(v) or v <= 0.0:
                raise ConfigError(f"Qwen3 `{key}` must be finite and positive, got {v}")
        if self.architectures and ARCHITECTURE not in self.architectures:
            raise ConfigError(f"Qwen3 config does not declare {ARCHITECTURE} (architectures = {list(self.architectures)})")
        if self.model_type is not None and self.model_type != "qwen3":
            raise ConfigError(f"Qwen3 config has model_type {self.model_type!r}, expected 'qwen3'")
        if self.use_sliding_window or self.sliding_window is not None:
            raise ConfigError("sliding-window attention is not part of Qwen3 dense as the reference runs it "
                              "(`use_sliding_window` must be false and `sliding_window` null)")
        if self.rope_scaling is not None:
            raise ConfigError("RoPE scaling is not supported (`rope_scaling` must be null)")
        if self.eos_token_id is not None and not 0 <= self.eos_token_id < self.vocab_size:
            raise ConfigError("eos_token_id is outside the vocabulary")

    # ---- the model as data --------------------------------------------

    def to_model_spec(self) -> ModelSpec:
        """Pre-norm decoder layers of GQA attention with per-head q/k norm and
        half-split rotary encoding, and a SiLU-gated feed-forward; the fixed
        choices (causal, scale head_dim^-1/2, rotary over the whole head, no
        biases) are the reference's (crates/quantinfer-model/src/qwen3.rs:135-250)."""
        d = self.effective_head_dim
        position = PositionSpec(head_dim=d, rotary_dim=d, theta=self.rope_theta,
                                max_positions=self.max_position_embeddings)
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            layers.append(LayerSpec(
                mixer_norm=NormSpec(self.hidden_size, self.rms_norm_eps, p + "input_layernorm."),
                mixer=AttentionSpec(
                    hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                    num_kv_heads=self.num_key_value_heads, head_dim=d, position=position,
                    qk_norm=True, qk_norm_eps=self.rms_norm_eps, window=None, scale=None,
                    prefix=p + "self_attn."),
                ffn_norm=NormSpec(self.hidden_size, self.rms_norm_eps, p + "post_attention_layernorm."),
                ffn=FeedForwardSpec(self.hidden_size, self.intermediate_size, "silu", p + "mlp."),
            ))
        spec = ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=EmbeddingSpec(self.vocab_size, self.hidden_size, "model.embed_tokens."),
            layers=tuple(layers),
            order=tuple(LayerCall(i, i) for i in range(self.num_hidden_layers)),
            final_norm=NormSpec(self.hidden_size, self.rms_norm_eps, "model.norm."),
            head=HeadSpec(self.vocab_size, self.hidden_size, self.tie_word_embeddings, "lm_head."),
            eos_token_id=self.eos_token_id,
        )
        spec.validate()
        return spec
