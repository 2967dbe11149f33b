"""A request and its sampling options (snowllm/engine/request.py:12-114: same names, same defaults,
same meanings; fields of speculation, images and prefix sharing are left out)."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..cache import RequestCache


@dataclass
class SamplingParams:
    temperature: float = 1.0            # <= 0: greedy
    top_p: float = 1.0
    top_k: int = 0                      # 0: no top-k cut
    max_new_tokens: int = 32
    stop_token_ids: tuple = ()
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    no_repeat_ngram_size: int = 0

    def penalized(self) -> bool:
        return bool(self.presence_penalty or self.frequency_penalty or self.repetition_penalty != 1.0)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


@dataclass(eq=False)
class Request:
    prompt: list
    params: SamplingParams
    out: list = field(default_factory=list)
    cache: RequestCache | None = None
    num_computed: int = 0               # tokens of ``tokens`` that are in the cache
    done: bool = False
    finish_reason: str | None = None    # "stop", "length", "abort", "error"
    error: str | None = None            # with finish_reason "error": what went wrong
    preemptions: int = 0
    arrival: int = 0                    # the engine's count of requests when this one was added
    in_flight: int = -1                 # >= 0: the last sampled token is still on the device, at this place
                                        # of the runner's pending tokens; the host has not read it yet

    @property
    def tokens(self) -> list:
        """Prompt and generated tokens; a token the host has not read yet appears as -(place + 1)."""
        if self.in_flight >= 0:
            return self.prompt + self.out + [-(self.in_flight + 1)]
        return self.prompt + self.out

    def tokens_at(self, start: int, count: int) -> list:
        """``tokens[start:start + count]`` without joining the lists (a decode step asks for one token of a
        request that may hold a hundred thousand)."""
        n, end = len(self.prompt), start + count
        if end <= n:
            return self.prompt[start:end]
        piece = self.prompt[start:n] if start < n else []
        lo = max(start - n, 0)
        piece = piece + self.out[lo:end - n]
        if self.in_flight >= 0 and end > n + len(self.out) and start <= n + len(self.out):
            piece = piece + [-(self.in_flight + 1)]
        return piece

    @property
    def generated(self) -> int:
        """Tokens sampled so far, the one in flight included."""
        return len(self.out) + (self.in_flight >= 0)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + self.generated

    @property
    def pending(self) -> int:
        """Tokens not yet run: the rest of the prompt, or the last sampled token."""
        return self.num_tokens - self.num_computed

    @property
    def at_length(self) -> bool:
        """The token in flight is the last one this request may generate: nothing more to schedule."""
        return self.generated >= self.params.max_new_tokens

    @property
    def last(self) -> int:
        return self.out[-1] if self.out else self.prompt[-1]
