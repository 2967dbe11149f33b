"""How a layer's parts sit around the residual stream.

``prenorm`` (snowllm/models/lfm2/layers.py:91-104): x += mixer(norm(x)); x += ffn(norm(x)).
The float residual sum is fused into the norm that follows it, so a block takes the delta that the
previous block left and returns its own last delta; the model adds the final one."""
from __future__ import annotations

from ..trace import span
from .registry import register_block


class PreNormBlock:
    def __init__(self, mixer, ffn, mixer_norm, ffn_norm):
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self._names = tuple(f"{what}:{type(part).__name__}" for what, part in
                            (("norm", mixer_norm), ("mixer", mixer), ("norm", ffn_norm), ("ffn", ffn)))

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def forward(self, ctx, residual, delta, cache, owns_cache=True):
        with span(self._names[0]):
            x = self.mixer_norm.forward(ctx, residual, delta)
        ctx.tap("mixer_in", x)
        with span(self._names[1]):
            delta = self.mixer.forward(ctx, x, cache, owns_cache)
        ctx.tap("mixer_out", delta)
        fused = getattr(self.ffn, "forward_from_residual", None)
        if fused is not None:          # a feed-forward that can take the norm before it into its first kernel
            with span(self._names[3]):
                out = fused(ctx, residual, delta, self.ffn_norm)
            if out is not None:
                ctx.tap("ffn_out", out)
                return out
        with span(self._names[2]):
            x = self.ffn_norm.forward(ctx, residual, delta)
        ctx.tap("ffn_in", x)
        with span(self._names[3]):
            delta = self.ffn.forward(ctx, x)
        ctx.tap("ffn_out", delta)
        return delta


register_block("prenorm", PreNormBlock)
