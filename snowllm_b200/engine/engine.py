"""The Engine: scheduler + cache manager + step function + sampler behind ``add / step / run``
(the interface of snowllm/engine/__init__.py:355-370, 604-709; Python use as in
tests/test_lfm2_e2e.py:16-27):

    model = snowllm_b200.load(path)
    engine = Engine(model, max_num_seqs=2, max_model_len=2048, stop_token_ids=stops, prefill_chunk=64)
    r = engine.add(ids, SamplingParams(temperature=0, max_new_tokens=256))
    engine.run()
    r.out, r.finish_reason
"""
from __future__ import annotations

import time
from dataclasses import asdict, dataclass, field

import torch

from ..cache import CacheManager, pages_for
from ..config.engine import (DEFAULT_GPU_UTIL, DEFAULT_MAX_NUM_SEQS, DEFAULT_PAGE_SIZE,
                             DEFAULT_PREFILL_CHUNK, MAX_NUM_SEQS)
from ..errors import CapacityError, SnowLLMError
from ..sampling import Sampler
from .request import Request, SamplingParams
from .runner import ModelRunner, StepEntry
from .scheduler import Scheduler


@dataclass
class StepAccounting:
    """Tokens, seconds and steps by kind of step (snowllm/engine/__init__.py:44-83)."""
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    prefill_steps: int = 0
    decode_tokens: int = 0
    decode_seconds: float = 0.0
    decode_steps: int = 0

    def add(self, prefill_tokens: int, decode_tokens: int, seconds: float) -> None:
        total = prefill_tokens + decode_tokens
        if prefill_tokens:
            self.prefill_tokens += prefill_tokens
            self.prefill_seconds += seconds * prefill_tokens / total
            self.prefill_steps += 1
        if decode_tokens:
            self.decode_tokens += decode_tokens
            self.decode_seconds += seconds * decode_tokens / total
            self.decode_steps += 1

    def snapshot(self) -> dict:
        d = asdict(self)
        d["prefill_tok_s"] = self.prefill_tokens / self.prefill_seconds if self.prefill_seconds else 0.0
        d["decode_tok_s"] = self.decode_tokens / self.decode_seconds if self.decode_seconds else 0.0
        return d


@dataclass
class EngineStats:
    """snowllm/engine/__init__.py:86-102 without the fields of prefix sharing and speculation."""
    running: int
    waiting: int
    free_slots: int
    free_kv_blocks: int
    preemptions: int
    steps: int
    accounting: dict = field(default_factory=dict)


class Engine:
    def __init__(self, model, num_kv_blocks: int | None = None, max_num_seqs: int = DEFAULT_MAX_NUM_SEQS,
                 max_model_len: int = 8192, stop_token_ids=(), seed: int | None = None,
                 enforce_eager: bool = False, prefill_chunk: int = DEFAULT_PREFILL_CHUNK,
                 gpu_memory_utilization: float = DEFAULT_GPU_UTIL, preempt: bool = True,
                 exact_stats: bool = False, page_size: int = DEFAULT_PAGE_SIZE, device="cuda",
                 overlap_steps: bool = True):
        if not 1 <= max_num_seqs <= MAX_NUM_SEQS:
            raise SnowLLMError(f"max_num_seqs must lie in 1..{MAX_NUM_SEQS}")
        self.model, self.device = model, torch.device(device)
        self.max_num_seqs, self.max_model_len = max_num_seqs, max_model_len
        self.enforce_eager, self.exact_stats = enforce_eager, exact_stats
        specs = model.cache_specs()
        if num_kv_blocks is None:
            # max_model_len is the shared capacity in tokens; one partial page per request on top
            num_kv_blocks = pages_for(max_model_len, page_size) + max_num_seqs
        per_page = sum(CacheManager.bytes_per_page(specs, page_size, model.dtype).values())
        free, total = torch.cuda.mem_get_info(self.device)
        budget = free - int(total * (1.0 - gpu_memory_utilization))
        if per_page * num_kv_blocks > budget:
            raise CapacityError(
                f"{num_kv_blocks} cache pages of {per_page} bytes need {per_page * num_kv_blocks >> 20} MiB, "
                f"the memory budget leaves {max(budget, 0) >> 20} MiB (gpu_memory_utilization="
                f"{gpu_memory_utilization}); lower max_model_len or num_kv_blocks")
        self.cache = CacheManager(specs, page_size, num_kv_blocks, max_num_seqs, model.dtype, self.device)
        self.runner = ModelRunner(model, self.cache, self.device, use_graphs=not enforce_eager)
        self.scheduler = Scheduler(self.cache, max_num_seqs, int(prefill_chunk), max_model_len, preempt)
        self.sampler = Sampler(stop_token_ids, seed, self.device)
        self.acct = StepAccounting()
        self.steps = 0
        self.overlap_steps = overlap_steps
        self._arrivals = 0
        self._flight = None                # (requests, pinned host tokens, event) of the step not yet read back
        self._landing = [torch.empty(MAX_NUM_SEQS, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._landing_turn = 0

    # -- the reference's names ------------------------------------------------------------
    @property
    def prefill_chunk(self) -> int:
        return self.scheduler.max_num_batched_tokens

    @prefill_chunk.setter
    def prefill_chunk(self, n: int) -> None:
        self.scheduler.max_num_batched_tokens = int(n)

    @property
    def waiting(self):
        return self.scheduler.waiting

    @property
    def running(self):
        return self.scheduler.running

    @property
    def stop_token_ids(self) -> frozenset:
        return self.sampler.stop_token_ids

    def add(self, prompt, params: SamplingParams | None = None) -> Request:
        r = Request(prompt=[int(t) for t in prompt], params=params or SamplingParams(), arrival=self._arrivals)
        self._arrivals += 1
        V = self.model.vocab_size
        if any(not 0 <= t < V for t in r.prompt):
            raise SnowLLMError(f"prompt holds a token id outside [0, {V})")
        self.scheduler.add(r)
        return r

    def abort(self, r: Request) -> None:
        self._land()
        r.in_flight = -1
        self.scheduler.abort(r)

    def step(self) -> str:
        """One scheduling round and one model step: "prefill", "decode", "mixed" or "idle" ("drain" when
        the round only read back the tokens of the step before).

        Overlapped steps (``overlap_steps``): the sampled tokens stay on the device, where the next step's
        embedding finds them, and reach the host one step late.  So the host plans and launches step k + 1
        while step k still runs; a request that ended on a stop token is found out one step late too, and
        the row it was given in between is thrown away.  Steps whose sampling looks at the generated tokens
        (penalties, n-gram bans), and steps in which pages could run out, first read everything back."""
        t0 = time.perf_counter()
        if self._flight is not None and self.cache.min_free_pages() < len(self.scheduler.running) + 1:
            self._land()                   # a decoding request might be preempted: its tokens must be known
        self.scheduler.retire_finished()
        plan = self.scheduler.schedule()
        if not plan:
            if self._flight is None:
                return "idle"
            self._land()
            return "drain"
        entries = [StepEntry(s.request.cache, s.tokens, [s.count - 1] if s.wants_logits else [])
                   for s in plan]
        decode = sum(1 for s in plan if s.count == 1 and s.start >= len(s.request.prompt))
        logits = self.runner.step(entries)
        for s in plan:
            s.request.num_computed += s.count
        self._land()                       # the step before: its tokens are on the host by now, or soon
        sampled = [s.request for s in plan if s.wants_logits]
        if sampled:
            if self.overlap_steps and not self.sampler.needs_history(sampled):
                self._take_off(logits, sampled)
            else:
                for r, tok in zip(sampled, self.sampler.sample(logits, sampled)):
                    if not r.done:
                        self.sampler.append(r, tok)
        if self.exact_stats:
            torch.cuda.synchronize(self.device)
        prefill = sum(s.count for s in plan) - decode
        self.acct.add(prefill, decode, time.perf_counter() - t0)
        self.steps += 1
        return "mixed" if prefill and decode else ("prefill" if prefill else "decode")

    def _take_off(self, logits, sampled) -> None:
        """Sample on the device into the runner's pending tokens and start their copy to the host."""
        n = len(sampled)
        self.sampler.sample_on_device(logits, sampled, out=self.runner.pending_tokens[:n])
        host = self._landing[self._landing_turn]
        self._landing_turn ^= 1
        host[:n].copy_(self.runner.pending_tokens[:n], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        for i, r in enumerate(sampled):
            if not r.done:                 # found out at the landing just before: the row is thrown away
                r.in_flight = i
        self._flight = (sampled, host, event)

    def _land(self) -> None:
        """Read back the tokens of the step in flight, if any, and record them."""
        if self._flight is None:
            return
        sampled, host, event = self._flight
        self._flight = None
        event.synchronize()
        tokens = host[:len(sampled)].tolist()
        for i, (r, tok) in enumerate(zip(sampled, tokens)):
            if r.in_flight == i and not r.done:
                r.in_flight = -1
                self.sampler.append(r, tok)

    def run(self) -> None:
        while self.scheduler.has_work():
            if self.step() == "idle":
                break
        self._land()
        self.scheduler.retire_finished()

    def generate(self, prompts, params: SamplingParams | None = None) -> list:
        """Token lists in, generated token lists out (a convenience over add + run)."""
        reqs = [self.add(p, params) for p in prompts]
        self.run()
        return [r.out for r in reqs]

    def stats(self) -> EngineStats:
        return EngineStats(running=len(self.running), waiting=len(self.waiting),
                           free_slots=self.cache.slots.free_count,
                           free_kv_blocks=self.cache.min_free_pages(),
                           preemptions=self.scheduler.preemptions, steps=self.steps,
                           accounting=self.acct.snapshot())
