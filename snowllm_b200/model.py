"""A model built from a ModelSpec: parts looked up by kind, run in the order the spec lists.

The forward pass works on one step's flat batch: embedding into a float residual stream, the run
list's blocks (each with the cache of its own entry, or of the entry it shares with), then the
final norm and the head on the rows whose logits are wanted only
(snowllm/models/lfm2/layers.py:107-131; snowllm/engine/qwen_runner.py:163-180)."""
from __future__ import annotations

import torch

from .errors import ConfigError
from .parts.registry import lookup
from .parts.spec import ModelSpec, PagedKVSpec, PartSpec
from .trace import span


def _make(family: str, spec: PartSpec, dtype):
    return lookup(family, spec.kind)(dtype, spec.names, **dict(spec.params))


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, config=None):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ConfigError(f"compute dtype {dtype} is not supported (float32 or bfloat16)")
        self.spec, self.dtype, self.config = spec, dtype, config
        self.embedding = _make("embedding", spec.embedding, dtype)
        self.blocks = []
        for layer in spec.layers:
            block_cls = lookup("block", layer.block)
            self.blocks.append(block_cls(_make("mixer", layer.mixer, dtype), _make("ffn", layer.ffn, dtype),
                                         _make("norm", layer.mixer_norm, dtype),
                                         _make("norm", layer.ffn_norm, dtype)))
        self.final_norm = _make("norm", spec.final_norm, dtype)
        self.head = _make("head", spec.head, dtype)
        self.run = list(spec.run)
        for i, entry in enumerate(self.run):
            if not 0 <= entry.layer < len(self.blocks):
                raise ConfigError(f"run entry {i} names layer {entry.layer}, the model has {len(self.blocks)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < i or self.run[entry.cache_of].cache_of is not None:
                    raise ConfigError(f"run entry {i} must share the cache of an earlier entry that owns one")
                mine = self.blocks[entry.layer].mixer.cache_spec()
                theirs = self.blocks[self.run[entry.cache_of].layer].mixer.cache_spec()
                if mine != theirs or not isinstance(mine, PagedKVSpec):
                    raise ConfigError(f"run entry {i} cannot read entry {entry.cache_of}'s cache: "
                                      f"{mine} against {theirs}")
        self.bound = False
        self.bound_bytes: dict = {}        # id(part) -> {local tensor name -> bytes on the device}, set by the loader

    # -- structure ------------------------------------------------------------------------
    def parts(self):
        yield self.embedding
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm
        yield self.head

    def libraries(self) -> list[str]:
        """csrc libraries this model's parts launch from (what a first call has to compile)."""
        seen: dict[str, None] = {}
        for p in self.parts():
            for lib in getattr(p, "libraries", ()):
                seen[lib] = None
        return list(seen)

    def declare(self, has):
        """[(part, TensorSpec)] in checkpoint order; a tensor named twice is declared once."""
        out, seen = [], set()
        for part in self.parts():
            for spec in part.declare(has):
                if spec.name in seen:
                    continue
                seen.add(spec.name)
                out.append((part, spec))
        return out

    def finish_binding(self) -> None:
        if getattr(self.head, "tied", False):
            self.head.bind({"weight": self.embedding.weight})
        self.bound = True

    def cache_specs(self) -> dict:
        """{run entry index -> cache spec} for the entries that own a cache."""
        out = {}
        for i, entry in enumerate(self.run):
            if entry.cache_of is None:
                spec = self.blocks[entry.layer].mixer.cache_spec()
                if spec is not None:
                    out[i] = spec
        return out

    def weight_bytes_per_step(self, picked: dict | None = None) -> int:
        """Bytes of weights one step reads: what each part of each run entry says it reads of the tensors
        it declared (a layer that the run list names twice is read twice), the final norm and the head.
        ``picked``: {run entry index -> experts picked in the step} for parts that read only those."""
        def of(part, n=None):
            return part.bytes_read(self.bound_bytes.get(id(part), {}), n)
        total = of(self.embedding) + of(self.final_norm) + of(self.head)
        for i, entry in enumerate(self.run):
            for part in self.blocks[entry.layer].parts():
                total += of(part, (picked or {}).get(i))
        return total

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    # -- forward --------------------------------------------------------------------------
    def forward(self, ctx, cache) -> torch.Tensor:
        """Float logits [len(ctx.logit_rows), vocab] of one step."""
        with span("embedding"):
            residual = self.embedding.forward(ctx)
        delta = None
        for i, entry in enumerate(self.run):
            owner = i if entry.cache_of is None else entry.cache_of
            with span(f"run[{i}]:layer{entry.layer}"):
                delta = self.blocks[entry.layer].forward(ctx, residual, delta, cache.view(owner, ctx.block_tables),
                                                         owns_cache=entry.cache_of is None)
        if ctx.num_logit_rows == 0:
            return torch.empty(0, self.spec.vocab_size, dtype=torch.float32, device=residual.device)
        with span("head"):
            x = self.final_norm.forward(ctx, residual, delta, rows=ctx.logit_rows)
            return self.head.forward(ctx, x)
