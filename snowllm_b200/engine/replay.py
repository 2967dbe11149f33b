"""Trace replay on top of the step function: requests by name, their next tokens, which logits.

It owns nothing but the map from request name to the request's cache handle; loading, the cache
manager, the step function and the kernels are the ones generation uses."""
from __future__ import annotations

import torch

from ..cache import CacheManager
from ..config.engine import DEFAULT_PAGE_SIZE
from ..errors import CapacityError
from ..loader import load
from ..ops import kernels
from .runner import ModelRunner, StepEntry

ROUND_TO = 64      # a request's token count is rounded up to this when the pool is sized


class Replay:
    def __init__(self, model, dtype: str, max_tokens: int, max_requests: int = 8,
                 page_size: int = DEFAULT_PAGE_SIZE, device="cuda", use_graphs: bool = False):
        """``model``: a model folder, or a model whose weights are bound already."""
        if ROUND_TO % page_size:
            raise ValueError(f"page_size {page_size} must divide {ROUND_TO}")
        self.model = model if hasattr(model, "forward") else load(model, dtype, device)
        num_pages = -(-max_tokens // ROUND_TO) * (ROUND_TO // page_size)
        self.cache = CacheManager(self.model.cache_specs(), page_size, num_pages, max_requests,
                                  self.model.dtype, device)
        self.runner = ModelRunner(self.model, self.cache, device, use_graphs=use_graphs)
        self.status = kernels.StatusWatch()
        self.live: dict = {}

    def step(self, entries, end=()):
        """Run one step of the trace; returns the wanted logits on the host (float32) or None."""
        batch = []
        for e in entries:
            rc = self.live.get(e["id"])
            if rc is None:
                rc = self.cache.admit()
                if rc is None:
                    raise CapacityError(f"no free slot for request {e['id']!r}")
                self.live[e["id"]] = rc
            tokens = list(e["tokens"])
            if not self.cache.ensure(rc, rc.num_tokens + len(tokens)):
                raise CapacityError(f"request {e['id']!r} needs more pages than --max-tokens leaves "
                                    f"({self.cache.free_pages()} free)")
            batch.append(StepEntry(rc, tokens, list(e.get("want", ()))))
        logits = self.runner.step(batch)
        self.status.peek()
        wanted = sum(len(b.want) for b in batch)
        result = logits.float().cpu() if wanted else None
        if not wanted:
            torch.cuda.current_stream().synchronize()
        self.status.check()                # a kernel that gave up waiting: raise rather than write wrong logits
        for name in end:
            rc = self.live.pop(name, None)
            if rc is not None:
                self.cache.free(rc)
        return result
