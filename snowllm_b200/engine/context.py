"""The step's flat batch as the kernels see it (the role of Batch and ForwardContext,
snowllm/engine/forward_context.py:45-172, and of prefill_batch, snowllm/engine/inputs.py:10-63).

A step is a list of segments, one per request in it: ``n`` next tokens of that request starting at
position ``start`` (= tokens already cached).  A decoded token is a segment with n = 1; prompt
portions of any length sit beside them.  All integer metadata is packed into one pinned host buffer
and copied to the device in one transfer."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepContext:
    dtype: torch.dtype
    device: torch.device
    M: int                         # rows (tokens) in the step
    B: int                         # segments (requests) in the step
    token_ids: torch.Tensor        # int32 [M]
    positions: torch.Tensor        # int32 [M] absolute position of each row
    row_seg: torch.Tensor          # int32 [M] segment of each row
    cu_seqlens: torch.Tensor       # int32 [B+1] first row of each segment
    seg_start: torch.Tensor        # int32 [B] tokens cached before this step (0: fresh request)
    seg_slot: torch.Tensor         # int32 [B] state slot of each segment's request
    logit_rows: torch.Tensor       # int32 [R] rows whose logits are wanted
    num_logit_rows: int
    block_tables: dict             # group key -> int32 [B, max_pages]
    page_size: int
    host_positions: np.ndarray     # the same facts on the host, for launch decisions
    host_seg_start: list = field(default_factory=list)
    host_seg_len: list = field(default_factory=list)
    memo: dict = field(default_factory=dict)     # what parts worked out for this step (launch plans, uploaded lists)
    capture_max_len: int | None = None           # a captured step: its launches must serve sequences up to this length
    taps: list | None = None       # when a list: parts append (name, tensor) of chosen intermediates
    pending_tokens: torch.Tensor | None = None   # int32 on the device: a token id -(i + 1) stands for entry i

    def tap(self, name: str, tensor) -> None:
        if self.taps is not None:
            self.taps.append((name, tensor))

    def scratch(self, nbytes: int) -> torch.Tensor:
        """Scratch bytes for one kernel launch (stream-ordered, from torch's caching allocator)."""
        return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=self.device)


class HostStaging:
    """A small ring of pinned int32 buffers; a buffer is reused only after the copy that read it
    has finished (the role of Staging, snowllm/engine/block_manager.py:72-104)."""

    def __init__(self, device, depth: int = 4):
        self.device, self.depth = device, depth
        self.buffers: list = [None] * depth
        self.events: list = [None] * depth
        self.turn = 0
        self.bytes_uploaded = 0
        self.mirrors: dict = {}        # group key -> int32 [slots, width]: host copy of the block tables

    def mirror(self, g: int, key, entries, width: int) -> np.ndarray:
        """The host copy of group ``key``'s block tables, one row per slot, brought up to date for the
        requests of ``entries`` (only entries that changed since the last step are written; holes of a
        window group read as page 0, which no kernel touches)."""
        m = self.mirrors.get(key)
        rows = max(e.cache.slot for e in entries) + 1
        width = max(width, max(len(e.cache.tables[key]) for e in entries))   # pages may be taken ahead of use
        if m is None or m.shape[0] < rows or m.shape[1] < width:
            new = np.zeros((max(rows, m.shape[0] if m is not None else 0),
                            max(2 * width, m.shape[1] if m is not None else 0)), dtype=np.int32)
            if m is not None:
                new[:m.shape[0], :m.shape[1]] = m
            self.mirrors[key] = m = new
        for e in entries:
            rc = e.cache
            table = rc.tables[key]
            if rc.synced.get("mirror") is not self:    # first time this mirror sees the request
                rc.synced.clear()
                rc.synced["mirror"] = self
            done = rc.synced.get(key, 0)
            if len(table) > done:
                m[rc.slot, done:len(table)] = np.maximum(np.asarray(table[done:], dtype=np.int64), 0)
            rc.synced[key] = len(table)
        return m

    def upload(self, host: np.ndarray, into: torch.Tensor | None = None) -> torch.Tensor:
        """Copy ``host`` to the device through a pinned buffer: into a new tensor, or into ``into``."""
        i = self.turn
        self.turn = (self.turn + 1) % self.depth
        n = host.size
        buf = self.buffers[i]
        if self.events[i] is not None:
            self.events[i].synchronize()
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1024) * 2, dtype=torch.int32).pin_memory()
            self.buffers[i] = buf
        buf[:n].numpy()[:] = host
        if into is not None:
            into[:n].copy_(buf[:n], non_blocking=True)
            dev = into
        else:
            dev = buf[:n].to(self.device, non_blocking=True)
        self.bytes_uploaded += n * 4
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return dev
