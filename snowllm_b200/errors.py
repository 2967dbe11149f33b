"""Error types of the engine (the role of snowllm/errors.py:7-16)."""


class SnowLLMError(RuntimeError):
    """A request, a configuration or a checkpoint that the engine refuses."""


class ConfigError(SnowLLMError):
    """config.json is missing keys or holds values no part can take."""


class WeightError(SnowLLMError):
    """The checkpoint's tensors do not match what the model declares."""


class CapacityError(SnowLLMError):
    """The cache pools cannot hold what a step or a request needs."""


class KernelError(SnowLLMError):
    """A CUDA launch failed, or a kernel refused a size it cannot take."""
