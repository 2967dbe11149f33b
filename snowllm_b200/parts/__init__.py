"""Parts a model is put together from, their specs and their registries."""
from .registry import (kinds, lookup, register_block, register_embedding, register_ffn, register_head,  # noqa: F401
                       register_mixer, register_norm, register_position)
from .spec import (LayerSpec, ModelSpec, PagedKVSpec, PartSpec, RunEntry, SlotStateSpec, TensorSpec)  # noqa: F401
