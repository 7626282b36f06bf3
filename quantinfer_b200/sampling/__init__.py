from .params import GenerationConfig
from .sampler import Sampler
from .slots import SLOT_WORDS, RequestSlots

__all__ = ["GenerationConfig", "Sampler", "RequestSlots", "SLOT_WORDS"]
