from .params import GenerationConfig
from .sampler import Sampler

__all__ = ["GenerationConfig", "Sampler"]
