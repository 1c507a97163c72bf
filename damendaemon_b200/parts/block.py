"""Block arrangements: how a layer's norms, mixer and feed-forward are wired.

'pre_norm': x = x + mixer(norm[0](x)); x = x + feed_forward(norm[1](x))  (damendaemon/gpt2.py:47-64).
'pre_norm_mixer': x = x + mixer(norm[0](x)), a layer without a feed-forward.
'parallel': y = norm[0](x); x = x + mixer(y) + feed_forward(y): one norm, both read its output, both results are added
to the float32 stream (by the epilogues of their last products, one after the other).
'pre_norm_shift': 'pre_norm' (or, with one norm, 'pre_norm_mixer') whose mixer reads s[t] = n[t] + (n[t-1] - n[t]) * mu
with n = norm[0](x) and mu one number per channel; n[t-1] of a sequence's first token is zero, and across steps it is kept
per request (a state named 'shift' at the layer's cache site).
"""
from __future__ import annotations

from ..cache.manager import RequestState
from .registry import register_arrangement
from .spec import TensorDecl


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


@register_arrangement("pre_norm_shift")
class ShiftedPreNormBlock:
    def __init__(self, spec, norms, mixer, feed_forward):
        if len(norms) not in (1, 2):
            raise ValueError(f"a shifted pre-norm block takes one norm (no feed-forward) or two, got {len(norms)}")
        if not spec.shift_weight:
            raise ValueError("a shifted pre-norm block needs the name of its shift weights")
        if not hasattr(norms[0], "forward_shifted"):
            raise ValueError("the norm before a shifted mixer must offer forward_shifted (the RMS norm does)")
        self.spec, self.norms, self.mixer, self.feed_forward = spec, list(norms), mixer, feed_forward
        self.shift = None

    def bind(self, weights):
        self.shift = weights[self.spec.shift_weight]

    @staticmethod
    def tensor_decls(spec):
        return [TensorDecl(spec.shift_weight, (spec.norms[0].width,), "vector")]

    @staticmethod
    def cache_needs(spec):
        return [RequestState((spec.norms[0].width,), "float32", name="shift")]

    def forward(self, x, ctx, cache, position):
        y = self.norms[0].forward_shifted(x, self.shift, cache.named["shift"], ctx)
        x = self.mixer.forward(y, x, ctx, cache, position)
        if len(self.norms) == 1:
            return x
        return self.feed_forward.forward(self.norms[1].forward(x), x, ctx)
