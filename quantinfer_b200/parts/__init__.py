from . import attention, block, embedding, ffn, norm, position  # noqa: F401  (registers the built-in kinds)
from .base import Part, Runtime, build_part, part_class, register_part
from .linear import Linear

__all__ = ["Part", "Runtime", "build_part", "part_class", "register_part", "Linear"]
