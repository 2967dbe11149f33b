"""Step function, scheduler and the Engine entry point."""
from .request import Request, SamplingParams  # noqa: F401
from .runner import ModelRunner, StepEntry  # noqa: F401
from .scheduler import Scheduler, Segment  # noqa: F401


def __getattr__(name):
    if name in ("Engine", "EngineStats", "StepAccounting"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
