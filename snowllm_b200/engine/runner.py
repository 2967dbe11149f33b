"""The one step function: a batch of (request, its next tokens) in, logits at the wanted places out.

It runs only the tokens it is given, as one batch, against the cache that earlier steps left, and
records afterwards that the requests' caches grew.  Prompt portions and single decoded tokens may
be mixed and cut anywhere (the role of runner.forward, snowllm/engine/runner.py:498-526, without
its split into prefill-only and decode-only batches)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..cache import CacheManager, RequestCache
from ..config.engine import DEFAULT_MAX_GRAPHS, MAX_NUM_SEQS
from ..errors import CapacityError, KernelError, SnowLLMError
from ..ops import kernels
from .context import HostStaging, StepContext
from .graphs import GraphCache


@dataclass
class StepEntry:
    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)   # places among ``tokens`` whose logits are asked


class ModelRunner:
    def __init__(self, model, cache: CacheManager, device="cuda", use_graphs: bool = False,
                 max_graphs: int = DEFAULT_MAX_GRAPHS, graph_ceiling_bytes: int | None = None):
        """``use_graphs``: steps that hold one token per request and want every row's logits (decode
        steps) are captured as CUDA graphs, one per (batch size, longest sequence rounded up to a power
        of two), and replayed (snowllm/engine/runner.py:498-526, 555-581); everything else runs launch
        by launch.  At most ``max_graphs`` captures are kept (the least recently used one goes), and
        none is made that would take the device memory in use past ``graph_ceiling_bytes``: such
        steps run launch by launch, as do all steps after a capture ran out of memory."""
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine runs on the GPU only")
        if not model.bound:
            raise SnowLLMError("the model has no weights bound")
        self.model, self.cache = model, cache
        self.device = torch.device(device)
        self.staging = HostStaging(self.device)
        # Tokens that were sampled on the device and that the host may not have read yet.  An entry's
        # token -(i + 1) stands for pending_tokens[i] (see the Engine's overlapped steps).
        self.pending_tokens = torch.zeros(MAX_NUM_SEQS, dtype=torch.int32, device=self.device)
        kernels.libraries_for(model.libraries())
        self.steps = 0
        self.tokens = 0
        self.taps = None       # set to a list to collect what parts tap (tests and debugging)
        self.use_graphs = use_graphs
        self.graphs = GraphCache(max_graphs, graph_ceiling_bytes, in_use=self._bytes_in_use,
                                 release=torch.cuda.empty_cache, oom_errors=(torch.OutOfMemoryError,))
        self.graph_pool = None
        self.graph_replays = 0
        self.eager_steps = 0

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch; returns float logits [wanted rows, vocab] in entry order, then ``want``
        order.  Every entry's pages must have been taken already (``CacheManager.ensure``).  The
        tensor may be overwritten by the next step."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return torch.empty(0, self.model.vocab_size, dtype=torch.float32, device=self.device)
        decode_only = all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        logits = None
        if self.use_graphs and decode_only and self.taps is None:
            logits = self._graph_step(entries)
        if logits is None:
            ctx = self.build_context(entries)
            with torch.no_grad():
                logits = self.model.forward(ctx, self.cache)
            self.eager_steps += 1
        for e in entries:
            self.cache.commit(e.cache, e.cache.num_tokens + len(e.tokens))
        self.steps += 1
        self.tokens += sum(len(e.tokens) for e in entries)
        return logits

    def build_context(self, entries: Sequence[StepEntry], **kw) -> StepContext:
        return build_context(entries, self.cache, self.model.dtype, self.device, self.staging,
                             self.model.vocab_size, self.model.spec.max_position, self.taps,
                             pending_tokens=self.pending_tokens, **kw)

    # -- decode steps as CUDA graphs ------------------------------------------------------------
    def _bytes_in_use(self) -> int:
        free, total = torch.cuda.mem_get_info(self.device)
        return total - free

    def _graph_step(self, entries):
        """Replay the capture that serves this step (made now, if there is room for it); None when the
        step has to run launch by launch."""
        P = self.cache.page_size
        B = len(entries)
        longest = max(e.cache.num_tokens + 1 for e in entries)
        # the table width and the number of key chunks are part of the captured launches: the longest
        # sequence is rounded up to a power of two so that one capture serves a range of lengths
        max_len = _pow2_at_least(longest)
        width = -(-max_len // P)
        key = (B, max_len)
        graph = self.graphs.get(key, lambda: self._capture(key, entries))
        if graph is None:
            return None
        graph.refresh(self.build_context(entries, max_pages=width, host_only=True))
        graph.graph.replay()
        self.graph_replays += 1
        return graph.logits

    def _capture(self, key, entries):
        import dataclasses
        B, max_len = key
        width = -(-max_len // self.cache.page_size)
        host = self.build_context(entries, max_pages=width, host_only=True)
        graph = CapturedDecode(torch.empty(host.size, dtype=torch.int32, device=self.device), self.staging)
        graph.refresh(host)
        ctx = self.build_context(entries, max_pages=width, into=graph.buffer, capture_max_len=max_len)
        # Warm-up outside the graph, so that nothing is created for the first time while capturing.
        # It must leave no trace: its state slots are the spare slot nobody owns; the keys and values
        # it writes are the ones the replay writes again.
        spare = torch.full_like(ctx.seg_slot, self.cache.slots.dummy)
        with torch.no_grad():
            self.model.forward(dataclasses.replace(ctx, seg_slot=spare, memo={}), self.cache)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        if self.graph_pool is None:
            self.graph_pool = torch.cuda.graph_pool_handle()
        with torch.no_grad(), torch.cuda.graph(g, pool=self.graph_pool):
            graph.logits = self.model.forward(ctx, self.cache)
        graph.graph = g
        return graph


def _pow2_at_least(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


class CapturedDecode:
    """A captured decode step: the device buffer its launches read their metadata from, the graph,
    and the logits tensor it writes (the role of GraphInputs, snowllm/engine/graphs.py:115-148)."""

    def __init__(self, buffer: torch.Tensor, staging: HostStaging):
        self.buffer, self.staging = buffer, staging
        self.graph = None
        self.logits = None

    def refresh(self, host: np.ndarray) -> None:
        self.staging.upload(host, into=self.buffer)


def build_context(entries: Sequence[StepEntry], cache: CacheManager, dtype, device, staging: HostStaging,
                  vocab_size: int, max_position: int = 1 << 30, taps=None, max_pages: int | None = None,
                  into: torch.Tensor | None = None, host_only: bool = False, capture_max_len: int | None = None,
                  pending_tokens: torch.Tensor | None = None):
    """Turn a step's entries into the flat batch on the device (one host-to-device copy).
    ``max_pages`` fixes the block-table width; ``into`` is a device buffer that already holds the
    packed metadata (no copy is made); ``host_only`` returns the packed host array instead."""
    P = cache.page_size
    V = vocab_size
    B = len(entries)
    lens = [len(e.tokens) for e in entries]
    starts = [e.cache.num_tokens for e in entries]
    M = sum(lens)
    seen = set()
    for e, n, s in zip(entries, lens, starts):
        if id(e.cache) in seen:
            raise SnowLLMError("a request appears twice in one step")
        seen.add(id(e.cache))
        if e.cache.freed:
            raise SnowLLMError("a freed request cannot be stepped")
        if s + n > max_position:
            raise SnowLLMError(f"position {s + n} exceeds the model's limit {max_position}")
        need = -(-(s + n) // P)
        for key, table in e.cache.tables.items():
            if len(table) < need:
                raise CapacityError("the step was given tokens whose pages were not taken")
            if key[1] is not None:                     # a window group's table may have holes
                first = max(0, s - key[1] + 1) // P
                if any(p < 0 for p in table[first:need]):
                    raise CapacityError("the step was given tokens whose pages were not taken")
    ids = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=M)
    # a negative id -(i + 1) names a token the device still holds (pending_tokens[i])
    lowest = -pending_tokens.numel() if pending_tokens is not None else 0
    if M and (ids.min() < lowest or ids.max() >= V):
        raise SnowLLMError(f"token id outside [0, {V})")
    cu = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(lens, out=cu[1:])
    row_seg = np.repeat(np.arange(B), lens)
    positions = np.arange(M) - np.repeat(cu[:-1], lens) + np.repeat(starts, lens)
    logit_rows = []
    for b, e in enumerate(entries):
        for w in e.want:
            if not 0 <= w < lens[b]:
                raise SnowLLMError(f"wanted place {w} is outside the entry's {lens[b]} tokens")
            logit_rows.append(int(cu[b]) + int(w))
    groups = list(cache.groups)
    needed_pages = max(1, -(-max(s + n for s, n in zip(starts, lens)) // P))
    if max_pages is None:
        max_pages = needed_pages
    elif max_pages < needed_pages:
        raise CapacityError(f"a block table of {max_pages} entries cannot hold {needed_pages} pages")
    slots = np.asarray([e.cache.slot for e in entries])
    tables = np.stack([staging.mirror(g, key, entries, max_pages)[slots, :max_pages] for g, key in enumerate(groups)]) \
        if groups else np.zeros((0, B, max_pages), dtype=np.int32)
    parts = [ids, positions, row_seg, cu, np.asarray(starts), slots,
             np.asarray(logit_rows, dtype=np.int64), tables.reshape(-1)]
    sizes = [p.size for p in parts]
    # each part starts on a 16-byte boundary
    offs, total = [], 0
    for s in sizes:
        offs.append(total)
        total += -(-s // 4) * 4
    host = np.zeros(total, dtype=np.int32)
    for p, o in zip(parts, offs):
        host[o:o + p.size] = p
    if host_only:
        return host
    dev = into if into is not None else staging.upload(host)
    view = lambda i: dev[offs[i]:offs[i] + sizes[i]]
    tab = view(7).view(len(groups), B, max_pages)
    return StepContext(
        dtype=dtype, device=device, M=M, B=B, token_ids=view(0), positions=view(1),
        row_seg=view(2), cu_seqlens=view(3), seg_start=view(4), seg_slot=view(5), logit_rows=view(6),
        num_logit_rows=len(logit_rows), block_tables={key: tab[g] for g, key in enumerate(groups)},
        page_size=P, host_positions=positions.astype(np.int64), host_seg_start=list(starts),
        host_seg_len=list(lens), taps=taps, pending_tokens=pending_tokens, capture_max_len=capture_max_len)
