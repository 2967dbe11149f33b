"""Named spans around the engine's step and each part's forward, for a timeline in a profiler
(the role of snowllm/trace.py:12-25).

Off by default: ``span`` then returns one shared do-nothing context and costs a dictionary lookup.
``SNOWLLM_B200_TRACE=1`` in the environment, ``enable()``, or a running ``torch.profiler`` session turn
every span into an NVTX range plus a ``record_function`` region; ``--enable-profiler`` on the command
line wraps the whole run in a ``torch.profiler`` session and writes a Chrome trace to ``--profile-dir``.
Spans are never opened while a CUDA graph is being captured (a captured step is one node on the timeline
anyway)."""
from __future__ import annotations

import contextlib
import os

_forced = os.environ.get("SNOWLLM_B200_TRACE", "") not in ("", "0")
_NULL = contextlib.nullcontext()


def enable(on: bool = True) -> None:
    global _forced
    _forced = bool(on)


def enabled() -> bool:
    if _forced:
        return True
    import torch
    return bool(torch.autograd._profiler_enabled())


@contextlib.contextmanager
def _region(name: str):
    import torch
    from torch.cuda import nvtx
    from torch.profiler import record_function
    if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        yield
        return
    with record_function(name), nvtx.range(name):
        yield


def span(name: str):
    """A context manager that names what runs inside it on the profiler's timeline."""
    return _region(name) if enabled() else _NULL


@contextlib.contextmanager
def profile_to(folder):
    """Run the body under ``torch.profiler`` (CPU and CUDA activity) and write ``trace.json`` into ``folder``."""
    import pathlib

    from torch.profiler import ProfilerActivity, profile
    folder = pathlib.Path(folder).expanduser()
    folder.mkdir(parents=True, exist_ok=True)
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        yield prof
    prof.export_chrome_trace(str(folder / "trace.json"))
