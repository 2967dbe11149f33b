"""snowllm_b200: a small, whole LFM2.5 inference engine for one B200 (sm_100a)."""
from .errors import CapacityError, ConfigError, KernelError, SnowLLMError, WeightError  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    # heavy modules load on first use, so that `import snowllm_b200` stays cheap
    if name in ("load", "load_random", "build_model"):
        from . import loader
        return getattr(loader, name)
    if name in ("Engine", "SamplingParams", "Request"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
