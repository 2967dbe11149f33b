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
from ..config.engine import MAX_NUM_SEQS, EngineConfig
from ..errors import CapacityError, KernelError, SnowLLMError
from ..ops import kernels
from ..sampling import Sampler
from ..trace import span
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
    step_errors: int = 0
    failed_requests: int = 0
    graphs: dict = field(default_factory=dict)


class Engine:
    def __init__(self, model, config: EngineConfig | None = None, device="cuda", runner=None, sampler=None,
                 status=None, **settings):
        """``config``, or the same settings as keyword arguments under SnowLLM's names (``max_num_seqs``,
        ``max_model_len``, ``prefill_chunk``, ``num_kv_blocks``, ``stop_token_ids``, ``seed``,
        ``enforce_eager``, ``gpu_memory_utilization``, ``preempt``, ``exact_stats``, ``page_size``,
        ``overlap_steps``, ``max_graphs``).  ``runner`` / ``sampler`` / ``status``: stand-ins for the step
        function, the sampler and the kernels' status words; with a ``runner`` given the engine touches
        no device itself and uses the runner's cache manager (how the host-side tests drive it)."""
        if config is not None and settings:
            raise SnowLLMError("give Engine a config or keyword settings, not both")
        self.config = c = config if config is not None else EngineConfig.from_kwargs(**settings)
        self.model, self.device = model, torch.device(device)
        self.max_num_seqs, self.max_model_len = c.max_num_seqs, c.max_model_len
        self.enforce_eager, self.exact_stats = c.enforce_eager, c.exact_stats
        if runner is None:
            specs = model.cache_specs()
            num_kv_blocks = c.num_kv_blocks
            if num_kv_blocks is None:
                # max_model_len is the shared capacity in tokens; one partial page per request on top
                num_kv_blocks = pages_for(c.max_model_len, c.page_size) + c.max_num_seqs
            per_page = sum(CacheManager.bytes_per_page(specs, c.page_size, model.dtype).values())
            free, total = torch.cuda.mem_get_info(self.device)
            ceiling = int(total * c.gpu_memory_utilization)
            budget = free - (total - ceiling)
            if per_page * num_kv_blocks > budget:
                raise CapacityError(
                    f"{num_kv_blocks} cache pages of {per_page} bytes need {per_page * num_kv_blocks >> 20} MiB, "
                    f"the memory budget leaves {max(budget, 0) >> 20} MiB (gpu_memory_utilization="
                    f"{c.gpu_memory_utilization}); lower max_model_len or num_kv_blocks")
            self.cache = CacheManager(specs, c.page_size, num_kv_blocks, c.max_num_seqs, model.dtype, self.device)
            self.runner = ModelRunner(model, self.cache, self.device, use_graphs=not c.enforce_eager,
                                      max_graphs=c.max_graphs, graph_ceiling_bytes=ceiling)
            self.sampler = sampler or Sampler(c.stop_token_ids, c.seed, self.device)
            self.status = status or kernels.StatusWatch()
            self._landing = [torch.empty(MAX_NUM_SEQS, dtype=torch.int32).pin_memory() for _ in range(2)]
        else:
            self.runner, self.cache = runner, runner.cache
            self.sampler = sampler or Sampler(c.stop_token_ids, c.seed, self.device)
            self.status = status
            self._landing = [torch.empty(MAX_NUM_SEQS, dtype=torch.int32) for _ in range(2)]
        self.scheduler = Scheduler(self.cache, c.max_num_seqs, c.max_num_batched_tokens, c.max_model_len,
                                   c.preempt)
        self.acct = StepAccounting()
        self.steps = 0
        self.step_errors = 0               # steps that failed: their requests ended with finish_reason "error"
        self.last_error: str | None = None
        self.overlap_steps = c.overlap_steps
        self._arrivals = 0
        self._flight = None                # (requests, pinned host tokens, event) of the step not yet read back
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
        the round only read back the tokens of the step before; "error" when the step failed).

        Overlapped steps (``overlap_steps``): the sampled tokens stay on the device, where the next step's
        embedding finds them, and reach the host one step late.  So the host plans and launches step k + 1
        while step k still runs; a request that ended on a stop token is found out one step late too, and
        the row it was given in between is thrown away.  Steps whose sampling looks at the generated tokens
        (penalties, n-gram bans), and steps in which pages could run out, first read everything back.

        A step that fails (an exception on the host, a kernel that reports a wait that ran out) ends the
        requests it touched with ``finish_reason == "error"``, gives back what they hold, records the
        reason in ``last_error`` and leaves the engine usable: waiting requests run in the next steps
        (snowllm/engine/async_engine.py:225-236, 283-286)."""
        t0 = time.perf_counter()
        plan = None
        try:
            with span("engine.step"):
                if self._flight is not None and self.cache.min_free_pages() < len(self.scheduler.running) + 1:
                    self._land()               # a decoding request might be preempted: its tokens must be known
                self.scheduler.retire_finished()
                plan = self.scheduler.schedule()
                if not plan:
                    if self._flight is None:
                        return "idle"
                    self._land()
                    return "drain"
                kind, prefill, decode = self._run(plan)
        except Exception as e:  # noqa: BLE001 - whatever went wrong, the engine goes on without these requests
            self._fail_step(e, plan)
            return "error"
        if self.exact_stats:
            torch.cuda.synchronize(self.device)
        self.acct.add(prefill, decode, time.perf_counter() - t0)
        self.steps += 1
        return kind

    def _run(self, plan):
        entries = [StepEntry(s.request.cache, s.tokens, [s.count - 1] if s.wants_logits else [])
                   for s in plan]
        decode = sum(1 for s in plan if s.count == 1 and s.start >= len(s.request.prompt))
        logits = self.runner.step(entries)
        for s in plan:
            s.request.num_computed += s.count
        if self.status is not None:
            self.status.peek()
        self._land()                       # the step before: its tokens are on the host by now, or soon
        sampled = [s.request for s in plan if s.wants_logits]
        if sampled:
            if self.overlap_steps and not self.sampler.needs_history(sampled):
                self._take_off(logits, sampled)
            else:
                tokens = self.sampler.sample(logits, sampled)      # reads back: the host is in step with the device
                if self.status is not None:
                    self.status.check()
                for r, tok in zip(sampled, tokens):
                    if not r.done:
                        self.sampler.append(r, tok)
        prefill = sum(s.count for s in plan) - decode
        return ("mixed" if prefill and decode else ("prefill" if prefill else "decode")), prefill, decode

    def _fail_step(self, e: Exception, plan) -> None:
        """End the requests a failed step touched; everything they hold comes back."""
        self.step_errors += 1
        self.last_error = why = f"{type(e).__name__}: {e}"
        flight, self._flight = self._flight, None
        hit = list(self.scheduler.running) if plan is None or isinstance(e, KernelError) \
            else [s.request for s in plan]
        if flight is not None:
            # tokens of the step before that the host has not read: read them if the device still answers
            try:
                self._flight = flight
                self._land()
            except Exception:  # noqa: BLE001
                self._flight = None
                hit += [r for i, r in enumerate(flight[0]) if r.in_flight == i]
        for r in hit:
            if not r.done or r.cache is not None:
                self.scheduler.fail(r, why)

    def _take_off(self, logits, sampled) -> None:
        """Sample on the device into the runner's pending tokens and start their copy to the host."""
        n = len(sampled)
        self.sampler.sample_on_device(logits, sampled, out=self.runner.pending_tokens[:n])
        host = self._landing[self._landing_turn]
        self._landing_turn ^= 1
        host[:n].copy_(self.runner.pending_tokens[:n], non_blocking=True)
        if self.status is not None:
            self.status.peek()
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
        if self.status is not None:
            self.status.check()
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
        """Counters of the engine.  ``accounting`` holds tokens, seconds and rates by kind of step; the
        seconds are device times only with ``exact_stats`` (every step then ends with a synchronise).
        Without it a step's time is the host's time to plan and launch it, which under overlapped steps
        is shorter than the device's: the rates then say how fast the host feeds the device."""
        return EngineStats(running=len(self.running), waiting=len(self.waiting),
                           free_slots=self.cache.slots.free_count,
                           free_kv_blocks=self.cache.min_free_pages(),
                           preemptions=self.scheduler.preemptions, steps=self.steps,
                           accounting=self.acct.snapshot(), step_errors=self.step_errors,
                           failed_requests=self.scheduler.failed,
                           graphs=self.runner.graphs.snapshot() if hasattr(self.runner, "graphs") else {})
