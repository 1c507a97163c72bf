"""Two mixers side by side: both read the same input; each output is divided by its root mean square over the model width
and multiplied by a weight, and ``factor`` times their sum is added to the stream.

The two are mixers of any registered kind, built from their own specs; they share the stop's cache site, so their cache
needs must not collide (at most one paged need, one state without a name, and names that differ). Each runs as it would
alone, with a stream of zeros in place of the residual: its last product's epilogue then leaves the bare result in float32.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import PagedNeed, RequestState
from .interfaces import Mixer
from .registry import MIXERS, lookup, register_mixer
from .spec import TensorDecl


def _both(spec):
    return ((spec.left, lookup(MIXERS, spec.left, "mixer")), (spec.right, lookup(MIXERS, spec.right, "mixer")))


@register_mixer("side_by_side")
class SideBySide(Mixer):
    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        self.left, self.right = (cls(sub, weights, runtime) for sub, cls in _both(spec))
        self.left_norm, self.right_norm = weights[spec.left_norm], weights[spec.right_norm]
        self.graph_safe = bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))
        self.portion_multiple = max(int(getattr(self.left, "portion_multiple", 1)), int(getattr(self.right, "portion_multiple", 1)))

    @staticmethod
    def tensor_decls(spec):
        decls = [d for sub, cls in _both(spec) for d in cls.tensor_decls(sub)]
        return decls + [TensorDecl(spec.left_norm, (spec.width,), "vector"), TensorDecl(spec.right_norm, (spec.width,), "vector")]

    @staticmethod
    def cache_needs(spec):
        needs = [n for sub, cls in _both(spec) for n in cls.cache_needs(sub)]
        paged = [n for n in needs if isinstance(n, PagedNeed)]
        names = [n.name for n in needs if isinstance(n, RequestState)]
        if len(paged) > 1 or len(set(names)) != len(names):
            raise ValueError("two mixers side by side share one cache site: at most one of them may keep pages, and their states "
                             f"must differ in name (pages: {len(paged)}, states: {names})")
        return needs

    def forward(self, y, residual, ctx, cache, position):
        both = torch.zeros((2, *residual.shape), dtype=torch.float32, device=residual.device)
        left = self.left.forward(y, both[0], ctx, cache, position)
        right = self.right.forward(y, both[1], ctx, cache, position)
        return kernels.norm_pair_add(residual, left, right, self.left_norm, self.right_norm, self.spec.norm_eps, self.spec.factor)
