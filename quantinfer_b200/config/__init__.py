from .qwen3 import Qwen3Config
from .registry import (architectures, config_class_for, config_from_dict, load_config,
                       register_architecture)
from .spec import (AttentionSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerCall, LayerSpec,
                   ModelSpec, NormSpec, PositionSpec)

__all__ = [
    "Qwen3Config", "architectures", "config_class_for", "config_from_dict", "load_config",
    "register_architecture", "AttentionSpec", "EmbeddingSpec", "FeedForwardSpec", "HeadSpec",
    "LayerCall", "LayerSpec", "ModelSpec", "NormSpec", "PositionSpec",
]
