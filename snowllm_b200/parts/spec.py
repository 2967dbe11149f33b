"""Data that describes a model: which parts, with which constants, in which order.

An architecture turns its typed configuration into a ``ModelSpec``.  Nothing in a
``ModelSpec`` is code: parts are named by the kind under which they are registered
(``parts.registry``), their sizes and constants are plain parameters, their weights
are named by checkpoint tensor name, and the order in which layers run is a list.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence

# How a tensor is filled by the random-weights mode.
INIT_NORMAL = "normal"      # N(0, std)
INIT_ONES = "ones"          # norm weights
INIT_CONV = "conv"          # N(0, conv_std)
INIT_BIAS = "bias"          # N(0, bias_std)

# How a tensor is kept on the device.
KEEP_COMPUTE = "compute"    # the engine's compute dtype (bfloat16, or float32 on the 32-bit path)
KEEP_SMALL = "small"        # stays float32 if the file stores it so, else the compute dtype
KEEP_F32 = "f32"            # always float32
KEEP_I32 = "i32"            # integer tables


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor that a part needs."""
    local: str                      # the part's own name for it
    name: str                       # checkpoint tensor name
    shape: tuple[int, ...]
    init: str = INIT_NORMAL
    keep: str = KEEP_COMPUTE
    file_shape: tuple[int, ...] | None = None   # shape as stored, when it differs (a view)

    @property
    def stored_shape(self) -> tuple[int, ...]:
        return self.file_shape if self.file_shape is not None else self.shape


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by kind, with its constants and its tensors' checkpoint names."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    names: Mapping[str, str] = field(default_factory=dict)   # local name or prefix -> checkpoint name


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged (block) and which parts they are."""
    block: str                      # arrangement kind, e.g. "prenorm"
    mixer: PartSpec
    ffn: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run list.  ``layer`` indexes ``ModelSpec.layers`` and may appear
    in several entries (shared weights).  ``cache_of`` names an earlier entry whose cache
    this entry reads instead of owning one (it then writes nothing into it)."""
    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: Sequence[LayerSpec]
    run: Sequence[RunEntry]
    final_norm: PartSpec
    head: PartSpec
    max_position: int = 1 << 30


# --- what a mixer asks of the cache manager -------------------------------------------

@dataclass(frozen=True)
class PagedKVSpec:
    """Rows that grow with the sequence, kept in pages.  ``window`` None keeps every row; an integer keeps
    the last ``window`` positions (the query's own included), so pages that fall wholly behind the window
    are given back.

    The spec chooses the layout of its pools (``pool_shapes``); the cache manager only makes them.
    Keys and values of one width lie in one tensor [pages, 2, kv heads, page_size, head_dim].  With
    ``v_head_dim`` of another width they are two tensors [pages, kv heads, page_size, width]; with
    ``v_head_dim`` 0 there is the key tensor alone (a latent row per position, a cache of keys only).
    ``cache_dtype`` None keeps the rows in the compute dtype; "float32" or "bfloat16" fixes it."""
    num_kv_heads: int
    head_dim: int
    window: int | None = None
    v_head_dim: int | None = None
    cache_dtype: str | None = None

    @property
    def fused(self) -> bool:
        return self.v_head_dim is None or self.v_head_dim == self.head_dim

    def pool_shapes(self, num_pages: int, page_size: int) -> tuple:
        if self.fused:
            return ((num_pages, 2, self.num_kv_heads, page_size, self.head_dim),)
        shapes = [(num_pages, self.num_kv_heads, page_size, self.head_dim)]
        if self.v_head_dim:
            shapes.append((num_pages, self.num_kv_heads, page_size, self.v_head_dim))
        return tuple(shapes)

    def elements_per_page(self, page_size: int) -> int:
        total = 0
        for shape in self.pool_shapes(1, page_size):
            n = 1
            for d in shape[1:]:
                n *= d
            total += n
        return total


@dataclass(frozen=True)
class SlotStateSpec:
    """State of fixed size per request: one tensor per shape, indexed by the request's slot.
    ``dtypes`` entries are "compute" or "f32"."""
    shapes: tuple[tuple[int, ...], ...]
    dtypes: tuple[str, ...] = ()
