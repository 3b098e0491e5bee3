"""Typed errors raised by the framework (all host-side)."""


class PicoError(Exception):
    """Base class of every error this package raises on purpose."""


class ConfigError(PicoError):
    """A config.json key is missing, has the wrong type, or asks for something unsupported."""


class WeightError(PicoError):
    """The tensors of a model folder do not match what the model needs."""


class OutOfPages(PicoError):
    """The page pool cannot hold what was asked for, even with nothing else running."""


class KernelError(PicoError):
    """A CUDA kernel refused its arguments (a size it does not take) or the extension is missing."""


class ScheduleError(PicoError):
    """A request cannot be admitted (too long for the model or the cache)."""
