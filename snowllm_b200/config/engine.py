"""Engine-level settings and their defaults (the role of snowllm/defaults.py:4-12 and of the
keyword arguments of Engine, snowllm/engine/__init__.py:356-370)."""
from __future__ import annotations

from dataclasses import dataclass

DEFAULT_PAGE_SIZE = 16                 # tokens per cache page
DEFAULT_GPU_UTIL = 0.9                 # fraction of device memory the engine may fill
DEFAULT_PREFILL_CHUNK = 8192           # token budget of one step (--max-num-batched-tokens)
MAX_NUM_SEQS = 256
DEFAULT_MAX_NUM_SEQS = 4
DEFAULT_CONTEXT_TARGET = 409600        # shared cache tokens the command line asks for by default


@dataclass(frozen=True)
class EngineConfig:
    page_size: int = DEFAULT_PAGE_SIZE
    num_kv_blocks: int | None = None           # pages per cache group; None: from the memory budget
    max_num_seqs: int = DEFAULT_MAX_NUM_SEQS
    max_model_len: int = 8192                  # shared cache tokens, and the cap of one request
    max_num_batched_tokens: int = DEFAULT_PREFILL_CHUNK
    gpu_memory_utilization: float = DEFAULT_GPU_UTIL
    enforce_eager: bool = False
    preempt: bool = True
    seed: int | None = None
