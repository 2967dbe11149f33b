"""Captured decode steps under a budget (the role of GraphBudget, snowllm/engine/graphs.py:36-92, and of
the fall back to launch-by-launch steps, snowllm/engine/runner.py:618-630).

A captured step holds device memory of its own (its metadata buffer, its scratch, its [B, vocab] float
logits), and there is one per (batch size, table width, key-chunk count).  Two limits keep that bounded:

* a count: with ``max_graphs`` captures alive, the least recently used one goes before a new one comes;
  what it held returns to the captures' common pool and serves the next capture;
* a ceiling in bytes of device memory in use: a capture is only tried while ``in_use() + the largest
  growth one capture has caused so far`` stays below it.  Past it, and after an out-of-memory error
  inside a capture, nothing more is captured (``full``): shapes without a capture run launch by launch.

The class knows nothing of CUDA: what captures, what measures memory and what an out-of-memory error is
are given to it, so its decisions are tested on the CPU."""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable


class GraphCache:
    def __init__(self, max_graphs: int, ceiling_bytes: int | None, in_use: Callable[[], int],
                 release: Callable[[], None] = lambda: None, oom_errors: tuple = (MemoryError,)):
        self.max_graphs, self.ceiling_bytes = max_graphs, ceiling_bytes
        self._in_use, self._release, self._oom = in_use, release, oom_errors
        self.entries: OrderedDict = OrderedDict()
        self.largest = 0           # the most bytes one capture has added to the memory in use
        self.full = False
        self.captures = 0
        self.evictions = 0
        self.refused = 0           # steps that asked for a capture and ran launch by launch instead

    def __len__(self) -> int:
        return len(self.entries)

    def get(self, key, capture: Callable[[], object]):
        """The capture of ``key``, made now if there is room; None when the step must run launch by launch."""
        hit = self.entries.get(key)
        if hit is not None:
            self.entries.move_to_end(key)
            return hit
        if self.full or self.max_graphs <= 0:
            self.refused += 1
            return None
        while len(self.entries) >= self.max_graphs:
            self.entries.popitem(last=False)
            self.evictions += 1
        before = self._in_use()
        if self.ceiling_bytes is not None and before + self.largest > self.ceiling_bytes:
            self.full = True
            self.refused += 1
            return None
        try:
            made = capture()
        except self._oom:
            # what the failed capture took is given back; the captures that exist stay usable
            self.full = True
            self.refused += 1
            self._release()
            return None
        self.largest = max(self.largest, self._in_use() - before)
        self.captures += 1
        self.entries[key] = made
        return made

    def clear(self) -> None:
        self.entries.clear()
        self._release()

    def snapshot(self) -> dict:
        return {"graphs": len(self.entries), "captures": self.captures, "evictions": self.evictions,
                "refused": self.refused, "full": self.full, "largest_bytes": self.largest}
