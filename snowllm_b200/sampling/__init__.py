"""Sampling: options per request, penalties, greedy and temperature / top-k / top-p draws."""
from .ngram import banned_ngram_tokens  # noqa: F401
from .sampler import Sampler  # noqa: F401
