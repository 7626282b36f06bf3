"""quantinfer_b200: a small, whole inference engine for one GPU (B200, sm_100a).

From a model folder (config.json + safetensors) to generated tokens: typed
configuration and an architecture registry, weights by name, layers composed
from parts, a paged cache manager, one step function, a scheduler, sampling,
hand-written CUDA kernels, and trace replay.
"""

from .api import EOS_AUTO, Model
from .errors import CacheError, ConfigError, KernelError, OutOfPages, QuantInferError, WeightError
from .sampling import GenerationConfig

__version__ = "0.1.0"

__all__ = ["EOS_AUTO", "Model", "GenerationConfig", "QuantInferError", "ConfigError", "WeightError",
           "KernelError", "CacheError", "OutOfPages", "__version__"]
