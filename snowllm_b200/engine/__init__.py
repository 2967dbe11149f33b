"""Step function, scheduler and the Engine entry point."""
from .runner import ModelRunner, StepEntry  # noqa: F401
