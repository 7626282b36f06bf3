"""Error types of the engine.

The reference separates invalid arguments from runtime failures at its C
boundary (status 1 -> ValueError, status 3 -> QuantInferError;
bindings/c/include/quantinfer.h:14-19, bindings/python/quantinfer/_ffi.py:77-84).
The same split is kept here as exception classes.
"""


class QuantInferError(RuntimeError):
    """A failure while loading or running a model."""


class ConfigError(ValueError):
    """config.json is missing a key, has a wrong type or fails validation."""


class WeightError(QuantInferError):
    """The weight files do not match what the model needs."""


class KernelError(QuantInferError):
    """A kernel refused its arguments, or the compiled kernels are missing."""


class CacheError(QuantInferError):
    """The cache manager was asked for something it cannot give."""


class OutOfPages(CacheError):
    """No free page is left in a layer group's pool."""
