"""How a layer's parts sit around the residual stream.

``prenorm`` (snowllm/models/lfm2/layers.py:91-104): x += mixer(norm(x)); x += ffn(norm(x)).
The float residual sum is fused into the norm that follows it, so a block takes the delta that the
previous block left and returns its own last delta; the model adds the final one."""
from __future__ import annotations

from .registry import register_block


class PreNormBlock:
    def __init__(self, mixer, ffn, mixer_norm, ffn_norm):
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def forward(self, ctx, residual, delta, cache, owns_cache=True):
        x = self.mixer_norm.forward(ctx, residual, delta)
        delta = self.mixer.forward(ctx, x, cache, owns_cache)
        x = self.ffn_norm.forward(ctx, residual, delta)
        return self.ffn.forward(ctx, x)


register_block("prenorm", PreNormBlock)
