"""Tokens that would complete an n-gram already seen (the rule of snowllm/ngram.py:4-14)."""
from __future__ import annotations


def banned_ngram_tokens(tokens, size: int) -> list:
    """With the last size-1 tokens as prefix: every token that followed the same prefix earlier."""
    if size <= 0 or len(tokens) + 1 < size:
        return []
    prefix = tuple(tokens[len(tokens) - (size - 1):]) if size > 1 else ()
    seen = set()
    for i in range(len(tokens) - size + 1):
        if tuple(tokens[i:i + size - 1]) == prefix:
            seen.add(tokens[i + size - 1])
    return sorted(seen)
