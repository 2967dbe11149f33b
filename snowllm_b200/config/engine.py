"""Engine-level settings and their defaults (the role of snowllm/defaults.py:4-12 and of the
keyword arguments of Engine, snowllm/engine/__init__.py:356-370).

``EngineConfig`` is what an ``Engine`` is built from: ``Engine(model, config)``, or
``Engine(model, max_num_seqs=..., prefill_chunk=...)`` with SnowLLM's own keyword names, which
``EngineConfig.from_kwargs`` turns into one.  It is validated once, here."""
from __future__ import annotations

from dataclasses import dataclass, fields

from ..errors import SnowLLMError

# Tokens per cache page.  64: a page of one kv head is then one 8 KB TMA box, and a 256-key chunk of the decode
# attention 8 boxes instead of 32 (measured against pages of 16: the 64-request decode step of the 8B-A1B sizes
# 5.62 -> 5.52 ms, of the dense 1.2B sizes at context 32,768 6.37 -> 6.03 ms; pages of 128 and 256 gain a little
# more there, but 256 is past what the tcgen05 prompt kernel takes, and 64 is what the replay tool's pool is
# counted in).
DEFAULT_PAGE_SIZE = 64
DEFAULT_GPU_UTIL = 0.9                 # fraction of device memory the engine may fill
DEFAULT_PREFILL_CHUNK = 8192           # token budget of one step (--max-num-batched-tokens)
MAX_NUM_SEQS = 256
DEFAULT_MAX_NUM_SEQS = 4
DEFAULT_CONTEXT_TARGET = 409600        # shared cache tokens the command line asks for by default
DEFAULT_MAX_GRAPHS = 64                # captured decode steps kept at a time (least recently used goes first)

# SnowLLM's keyword names for the same settings
_ALIASES = {"prefill_chunk": "max_num_batched_tokens"}


@dataclass(frozen=True)
class EngineConfig:
    page_size: int = DEFAULT_PAGE_SIZE
    num_kv_blocks: int | None = None           # pages per cache group; None: from max_model_len
    max_num_seqs: int = DEFAULT_MAX_NUM_SEQS
    max_model_len: int = 8192                  # shared cache tokens, and the cap of one request
    max_num_batched_tokens: int = DEFAULT_PREFILL_CHUNK
    gpu_memory_utilization: float = DEFAULT_GPU_UTIL
    enforce_eager: bool = False                # no CUDA graphs for decode steps
    max_graphs: int = DEFAULT_MAX_GRAPHS
    preempt: bool = True
    seed: int | None = None
    stop_token_ids: tuple = ()
    overlap_steps: bool = True                 # sampled tokens stay on the device for one step
    exact_stats: bool = False                  # synchronise every step, so that step times are device times

    def __post_init__(self):
        problems = []
        if not 1 <= self.max_num_seqs <= MAX_NUM_SEQS:
            problems.append(f"max_num_seqs={self.max_num_seqs} must lie in 1..{MAX_NUM_SEQS}")
        if self.page_size < 1:
            problems.append(f"page_size={self.page_size} must be positive")
        if self.max_model_len < 1:
            problems.append(f"max_model_len={self.max_model_len} must be positive")
        if self.max_num_batched_tokens < 1:
            problems.append(f"max_num_batched_tokens={self.max_num_batched_tokens} must be positive")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            problems.append(f"gpu_memory_utilization={self.gpu_memory_utilization} must lie in (0, 1]")
        if self.num_kv_blocks is not None and self.num_kv_blocks < 1:
            problems.append(f"num_kv_blocks={self.num_kv_blocks} must be positive")
        if self.max_graphs < 0:
            problems.append(f"max_graphs={self.max_graphs} must not be negative")
        if problems:
            raise SnowLLMError("engine settings: " + "; ".join(problems))

    @classmethod
    def from_kwargs(cls, **kw) -> "EngineConfig":
        known = {f.name for f in fields(cls)}
        out = {}
        for k, v in kw.items():
            name = _ALIASES.get(k, k)
            if name not in known:
                raise SnowLLMError(f"Engine has no setting {k!r} (known: {', '.join(sorted(known | set(_ALIASES)))})")
            if name in ("max_num_batched_tokens", "max_model_len", "page_size", "max_num_seqs", "max_graphs"):
                v = int(v)
            if name == "stop_token_ids":
                v = tuple(v)
            out[name] = v
        return cls(**out)
