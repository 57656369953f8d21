"""Block arrangements: how a layer's norms, mixer and feed-forward are wired.

'pre_norm': x = x + mixer(norm[0](x)); x = x + feed_forward(norm[1](x))  (damendaemon/gpt2.py:47-64).
'pre_norm_mixer': x = x + mixer(norm[0](x)), a layer without a feed-forward.
'parallel': y = norm[0](x); x = x + mixer(y) + feed_forward(y): one norm, both read its output, both results are added
to the float32 stream (by the epilogues of their last products, one after the other).
"""
from __future__ import annotations

from .registry import register_arrangement


@register_arrangement("pre_norm")
class PreNormBlock:
    def __init__(self, spec, norms, mixer, feed_forward):
        if len(norms) != 2:
            raise ValueError(f"a pre-norm block takes two norms (before the mixer, before the feed-forward), got {len(norms)}")
        self.spec, self.norms, self.mixer, self.feed_forward = spec, list(norms), mixer, feed_forward

    def forward(self, x, ctx, cache, position):
        x = self.mixer.forward(self.norms[0].forward(x), x, ctx, cache, position)
        return self.feed_forward.forward(self.norms[1].forward(x), x, ctx)


@register_arrangement("pre_norm_mixer")
class PreNormMixerOnly:
    def __init__(self, spec, norms, mixer, feed_forward):
        if len(norms) != 1:
            raise ValueError(f"a mixer-only block takes one norm, got {len(norms)}")
        self.spec, self.norms, self.mixer, self.feed_forward = spec, list(norms), mixer, feed_forward

    def forward(self, x, ctx, cache, position):
        return self.mixer.forward(self.norms[0].forward(x), x, ctx, cache, position)


@register_arrangement("parallel")
class ParallelBlock:
    def __init__(self, spec, norms, mixer, feed_forward):
        if len(norms) != 1:
            raise ValueError(f"a parallel block takes one norm, got {len(norms)}")
        self.spec, self.norms, self.mixer, self.feed_forward = spec, list(norms), mixer, feed_forward

    def forward(self, x, ctx, cache, position):
        y = self.norms[0].forward(x)
        x = self.mixer.forward(y, x, ctx, cache, position)
        return self.feed_forward.forward(y, x, ctx)
