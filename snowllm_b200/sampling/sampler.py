"""From logits to tokens: penalties, n-gram bans, then argmax or a temperature / top-k / top-p draw
(snowllm/engine/sampler.py:86-104, 187-219, 229-234).  The arithmetic runs in csrc/sampling.cu on
float logits; this class gathers each row's options and the tokens its request has seen."""
from __future__ import annotations

import os
from collections import Counter

import numpy as np
import torch

from ..ops import kernels
from .ngram import banned_ngram_tokens


class Sampler:
    def __init__(self, stop_token_ids=(), seed: int | None = None, device="cuda"):
        self.stop_token_ids = frozenset(stop_token_ids)
        self.device = torch.device(device)
        self.seed = int(seed) if seed is not None else int.from_bytes(os.urandom(8), "little")

    def _i32(self, values):
        return torch.tensor(np.asarray(values, dtype=np.int32), device=self.device)

    def _f32(self, values):
        return torch.tensor(np.asarray(values, dtype=np.float32), device=self.device)

    def _penalize(self, logits, rows) -> None:
        offsets, ids, counts = [0], [], []
        for r in rows:
            p = r.params
            row_ids, row_counts = [], []
            if p.penalized():
                out_counts = Counter(r.out)
                seen = sorted(set(r.prompt) | out_counts.keys())
                row_ids += seen
                row_counts += [out_counts.get(t, 0) for t in seen]
            if p.no_repeat_ngram_size:
                banned = set(banned_ngram_tokens(r.tokens, p.no_repeat_ngram_size))
                # a banned token's entry replaces its penalty entry: ids of a row stay distinct
                keep = [(t, c) for t, c in zip(row_ids, row_counts) if t not in banned]
                row_ids = [t for t, _ in keep] + sorted(banned)
                row_counts = [c for _, c in keep] + [-1] * len(banned)
            ids += row_ids
            counts += row_counts
            offsets.append(len(ids))
        if not ids:
            return
        kernels.apply_penalties(
            logits, self._i32(offsets), self._i32(ids), self._i32(counts),
            self._f32([r.params.presence_penalty for r in rows]),
            self._f32([r.params.frequency_penalty for r in rows]),
            self._f32([r.params.repetition_penalty for r in rows]))

    def uniform(self, r) -> float:
        """The uniform number in [0, 1) behind a request's next token: a hash of the seed, the request's
        arrival number and how many tokens it has generated.  A request's draws therefore do not depend on
        what else is in the batch or on how the steps were cut."""
        mask = (1 << 64) - 1
        x = (self.seed + 0x9E3779B97F4A7C15 * (r.arrival + 1) + 0xD1B54A32D192ED03 * (r.generated + 1)) & mask
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & mask       # the splitmix64 finaliser
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & mask
        x ^= x >> 31
        return (x >> 40) / float(1 << 24)

    @staticmethod
    def needs_history(rows) -> bool:
        """Whether a row's options look at the tokens its request has generated (penalties, bans)."""
        return any(r.params.penalized() or r.params.no_repeat_ngram_size for r in rows)

    def sample_on_device(self, logits: torch.Tensor, rows, out: torch.Tensor | None = None) -> torch.Tensor:
        """One token per row of float logits [len(rows), V], left on the device (int32 [len(rows)])."""
        if self.needs_history(rows):
            self._penalize(logits, rows)
        if all(r.params.greedy for r in rows):
            return kernels.argmax(logits, out=out)
        uniform = self._f32([self.uniform(r) for r in rows])
        return kernels.sample(
            logits, self._f32([r.params.temperature for r in rows]),
            self._i32([max(0, r.params.top_k) for r in rows]),
            self._f32([r.params.top_p for r in rows]), uniform, out=out)

    def sample(self, logits: torch.Tensor, rows) -> list:
        """One token per row of float logits [len(rows), V]; ``rows`` are the requests."""
        if not rows:
            return []
        return self.sample_on_device(logits, rows).cpu().tolist()

    def append(self, r, token: int) -> None:
        """Record a sampled token and decide whether the request is finished."""
        r.out.append(int(token))
        if token in self.stop_token_ids or token in r.params.stop_token_ids:
            r.done, r.finish_reason = True, "stop"
        elif len(r.out) >= r.params.max_new_tokens:
            r.done, r.finish_reason = True, "length"
