"""What every part is: constants as constructor parameters, weights declared by checkpoint
name, bound once they are on the device, and a forward over the step's flat batch.

Interfaces (duck-typed; these base classes only hold what is common):

* every part:  ``__init__(dtype, names, **params)``, ``declare(has) -> [TensorSpec]``,
  ``bind(tensors)``; ``libraries`` names the csrc sources its kernels come from.
* mixer:       ``cache_spec() -> PagedKVSpec | SlotStateSpec | None`` and
               ``forward(ctx, x[M,H], cache, owns_cache) -> float delta [M,H]``
* feed-forward ``forward(ctx, x[M,H]) -> float delta [M,H]`` (or a ``kernels.ExpertSum``, a delta still in
               pieces that norms add up themselves; ``.dense()`` gives the tensor)
               Optional: ``forward_from_residual(ctx, residual, delta, norm) -> delta | None``: the norm
               before the feed-forward taken into its first kernel (None: not for this step or this norm;
               the block then calls the norm and ``forward``).  It must give what the two calls give.
* norm:        ``forward(ctx, residual, delta, rows=None) -> x[M,H]`` (adds delta into the float
               residual, then normalises into the compute dtype).  A norm that is x * rsqrt(mean(x^2) + eps)
               * weight over the whole width says so with ``fusable_rms = True`` (and ``weight``, ``eps``).
* position:    ``rotary(device) -> (inv_freq float [rot_dim/2] | None, rot_dim)``
* block:       ``forward(ctx, residual, delta, cache, owns_cache) -> delta`` (how mixer, feed-
               forward and norms are arranged around the residual stream)

No part knows which model it is in: what it needs comes through its parameters, its tensors
and the step context.
"""
from __future__ import annotations

from typing import Callable, Mapping

import torch

from .spec import TensorSpec


class Part:
    libraries: tuple[str, ...] = ()

    def __init__(self, dtype: torch.dtype, names: Mapping[str, str]):
        self.dtype = dtype
        self.names = dict(names)

    def declare(self, has: Callable[[str], bool]) -> list[TensorSpec]:
        """The checkpoint tensors this part needs; ``has(name)`` tells which spellings exist."""
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Take the loaded tensors (keyed by TensorSpec.local), fuse or reshape as needed."""

    def parts(self):
        """Parts nested in this one (their tensors are declared and bound through it)."""
        return ()

    def bytes_read(self, bound: Mapping[str, int], picked: int | None = None) -> int:
        """Bytes of its weights that one step reads, for roofline arithmetic.  ``bound``: {local tensor name ->
        bytes as kept on the device} of what this part declared.  The default is every tensor once; a part
        that reads only some of its weights (routed experts: ``picked`` of them were chosen in the step)
        says so here."""
        return sum(bound.values())
