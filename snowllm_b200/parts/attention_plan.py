"""Launch planning of the attention mixer: which rows go to which kernel, and into how many chunks of
keys a row's sequence is cut.  It reads the step's host-side facts (segment starts and lengths, row
positions) from the step context and keeps what it worked out in the context's per-step ``memo``, so
that the attention layers of one step plan (and upload their tile lists) once.  Another paged mixer
with other tile sizes brings a module like this one; the step context knows nothing of either."""
from __future__ import annotations

import numpy as np
import torch

ATTENTION_CHUNK = 256          # keys per block along the sequence when rows are few
ATTENTION_ROWS_ENOUGH = 128    # from this many rows on, rows alone fill the GPU: one chunk
ATTENTION_TILE = 32
PREFILL_MIN_ROWS = 16          # portions of at least this many rows go to the tensor-core prompt kernel
WHOLE = (1 << 30) - ((1 << 30) % ATTENTION_TILE)     # a chunk length that no sequence reaches


def prefill_tiles(seg_start, seg_len, tile_rows: int, min_rows: int = PREFILL_MIN_ROWS):
    """Split a step's rows between the prompt kernel and the row-wise kernel.  Returns
    (tiles [[segment, first row, rows, first position], ...], other rows [row, ...])."""
    tiles, rows, first = [], [], 0
    for b, (start, n) in enumerate(zip(seg_start, seg_len)):
        if n >= min_rows:
            for r in range(0, n, tile_rows):
                tiles.append([b, first + r, min(tile_rows, n - r), start + r])
        else:
            rows.extend(range(first, first + n))
        first += n
    return tiles, rows


def split(ctx, tile_rows: int):
    """(tiles int32 [n, 4] | None, other rows int32 [m] | None, host list of the other rows) for
    the prompt kernel and the row-wise kernel; uploaded once per step."""
    key = ("attention_split", tile_rows)
    if key not in ctx.memo:
        tiles, rows = prefill_tiles(ctx.host_seg_start, ctx.host_seg_len, tile_rows)
        dev_tiles = dev_rows = None
        if tiles:
            flat = torch.tensor(tiles, dtype=torch.int32).reshape(-1)
            both = torch.cat((flat, torch.tensor(rows, dtype=torch.int32)))
            both = both.pin_memory().to(ctx.device, non_blocking=True)
            dev_tiles = both[:flat.numel()].view(-1, 4)
            dev_rows = both[flat.numel():] if rows else None
        ctx.memo[key] = (dev_tiles, dev_rows, rows)
    return ctx.memo[key]


def _positions(ctx, rows):
    return ctx.host_positions if rows is None else ctx.host_positions[np.asarray(rows, dtype=np.int64)]


def chunks(ctx, window=None, rows=None, chunk: int = ATTENTION_CHUNK) -> int:
    """The most chunks of ``chunk`` keys that a row (of ``rows``, or of the step) spans.  A captured
    step is planned for the longest sequence its launches may ever serve."""
    if ctx.capture_max_len is not None:
        return max(1, -(-ctx.capture_max_len // chunk))
    pos = _positions(ctx, rows)
    if len(pos) == 0:
        return 1
    lo = np.maximum(0, pos - window + 1) if window else np.zeros_like(pos)
    return int((pos // chunk - lo // chunk).max()) + 1


def plan(ctx, window=None, rows=None) -> tuple[int, int]:
    """(chunk, num_chunks) for the row-wise kernel: with many rows one chunk per row, else chunks of
    ATTENTION_CHUNK keys so that long sequences spread over the GPU."""
    key = ("attention_plan", window, None if rows is None else len(rows))
    got = ctx.memo.get(key)
    if got is None:
        if ctx.capture_max_len is not None:
            got = (ATTENTION_CHUNK, chunks(ctx))           # a captured step: always chunks, of a fixed count
        else:
            pos = _positions(ctx, rows)
            if len(pos) >= ATTENTION_ROWS_ENOUGH or int(pos.max(initial=0)) < 2 * ATTENTION_CHUNK:
                got = (WHOLE, 1)
            else:
                n = chunks(ctx, window, rows)
                got = (ATTENTION_CHUNK, n) if n > 1 else (WHOLE, 1)
        ctx.memo[key] = got
    return got
