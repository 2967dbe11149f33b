"""The scheduler: which requests run which of their tokens in the next step.

Per step, under the token budget ``max_num_batched_tokens``: first one token for every running
request that is decoding, then portions of the prompts of running requests that are still being
prefilled (oldest first; a portion is whatever is left of the budget), then new admissions.
Admission takes a state slot and the pages of the whole prompt (snowllm/engine/__init__.py:723-765).
When a decoding request cannot get its next page, the most recently admitted running request is
preempted: everything it holds is given back, it returns to the front of the waiting queue, and on
re-admission it is prefilled again over its prompt and the tokens it had generated
(snowllm/engine/__init__.py:783-829).

A request that the pool could not hold even alone (its prompt and all the tokens it may generate) is
refused when it is added: CapacityError, and nothing else is touched.  What can still go wrong inside
a round (preemption switched off and no page left; a lone request that the pool has no page for)
ends that one request with ``finish_reason == "error"`` and the reason in ``Request.error``; the
others go on.  When the token budget is smaller than the number of decoding requests, the decode
pass starts each round where the last one stopped, so that every request gets its turn.

The scheduler does the book-keeping only; it never touches the device."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass

from ..cache import CacheManager
from ..errors import CapacityError, SnowLLMError
from .request import Request


@dataclass
class Segment:
    request: Request
    start: int              # position of the first token
    count: int              # tokens to run
    wants_logits: bool      # the segment reaches the end of the request's tokens

    @property
    def tokens(self) -> list:
        return self.request.tokens_at(self.start, self.count)


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int,
                 max_model_len: int, preempt: bool = True):
        if max_num_batched_tokens < 1:
            raise ValueError("max_num_batched_tokens must be at least 1")
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.preempt = preempt
        self.waiting: deque = deque()
        self.running: list = []
        self.preemptions = 0
        self.failed = 0                # requests ended with finish_reason "error" by the scheduler
        self._decode_turn = 0          # where the decode pass starts when the budget cannot serve everyone

    def add(self, r: Request) -> None:
        if not r.prompt:
            raise SnowLLMError("a request needs at least one prompt token")
        if len(r.prompt) + r.params.max_new_tokens > self.max_model_len:
            raise SnowLLMError(f"prompt {len(r.prompt)} + {r.params.max_new_tokens} new > "
                               f"max_model_len {self.max_model_len}")
        life = len(r.prompt) + r.params.max_new_tokens
        short = {k: (n, self.cache.groups[k].total) for k, n in self.cache.pages_for_life(life).items()
                 if n > self.cache.groups[k].total}
        if short:
            raise CapacityError(
                f"the cache cannot hold this request even alone: {life} tokens (prompt {len(r.prompt)} + "
                f"{r.params.max_new_tokens} new) need " +
                ", ".join(f"{n} pages of group {k} (it has {have})" for k, (n, have) in short.items()) +
                f" of page size {self.cache.page_size}; raise max_model_len or num_kv_blocks")
        self.waiting.append(r)

    def retire_finished(self) -> list:
        """Give back what finished requests hold; returns them."""
        gone = [r for r in self.running if r.done]
        for r in gone:
            self._release(r)
        self.running = [r for r in self.running if not r.done]
        return gone

    def abort(self, r: Request) -> None:
        if r in self.waiting:
            self.waiting.remove(r)
        elif r in self.running:
            self.running.remove(r)
            self._release(r)
        r.done, r.finish_reason = True, "abort"

    def _release(self, r: Request) -> None:
        if r.cache is not None:
            self.cache.free(r.cache)
            r.cache = None

    def fail(self, r: Request, why: str) -> None:
        """End one request with finish_reason "error": it gives everything back, the others go on."""
        if r in self.waiting:
            self.waiting.remove(r)
        elif r in self.running:
            self.running.remove(r)
        self._release(r)
        r.in_flight = -1
        r.done, r.finish_reason, r.error = True, "error", why
        self.failed += 1

    def _preempt_last(self) -> Request:
        victim = self.running.pop()
        self._release(victim)
        victim.num_computed = 0
        victim.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(victim)
        return victim

    def schedule(self) -> list:
        """The next step's segments (decoding requests first), or [] when there is nothing to do."""
        budget = self.max_num_batched_tokens
        plan: list = []
        # 1. one token for every decoding request; with a budget below their number, in turns
        decoders = [r for r in self.running
                    if not (r.done or r.at_length or r.pending != 1 or not r.generated)]
        if len(decoders) > budget:
            first = self._decode_turn % len(decoders)
            decoders = decoders[first:] + decoders[:first]
            self._decode_turn = first + budget
        for r in decoders:
            if budget <= 0:
                break
            if r.cache is None:                        # preempted for an earlier request of this pass
                continue
            while not self.cache.ensure(r.cache, r.num_computed + 1):
                if not self.preempt:
                    self.fail(r, "the cache is full and preemption is off")
                    break
                if len(self.running) == 1:
                    self.fail(r, f"the cache cannot hold one request of {r.num_computed + 1} tokens: "
                                 f"{self.cache.free_pages()} pages free")
                    break
                victim = self._preempt_last()
                plan = [s for s in plan if s.request is not victim]
                if victim is r:
                    break
            else:
                plan.append(Segment(r, r.num_computed, 1, True))
                budget -= 1
        # 2. prompt portions of running requests (their pages were taken at admission)
        for r in self.running:
            if budget <= 0:
                break
            if r.done or any(s.request is r for s in plan) or r.pending < 1 or (r.pending == 1 and r.generated):
                continue
            n = min(r.pending, budget)
            plan.append(Segment(r, r.num_computed, n, r.num_computed + n == r.num_tokens))
            budget -= n
        # 3. admissions
        while budget > 0 and self.waiting and len(self.running) < self.max_num_seqs:
            r = self.waiting[0]
            rc = self.cache.admit()
            if rc is None:
                break
            total = len(r.prompt) + len(r.out)
            if not self.cache.ensure(rc, total):
                self.cache.free(rc)
                if not self.running:
                    self.fail(r, f"the cache cannot admit a request of {total} tokens with nothing else "
                                 f"running: {self.cache.free_pages()} pages free of page size "
                                 f"{self.cache.page_size}")
                    continue
                break
            self.waiting.popleft()
            r.cache, r.num_computed = rc, 0
            self.running.append(r)
            n = min(total, budget)
            plan.append(Segment(r, 0, n, n == total))
            budget -= n
        return plan

    def has_work(self) -> bool:
        return bool(self.waiting) or any(not r.done for r in self.running)
