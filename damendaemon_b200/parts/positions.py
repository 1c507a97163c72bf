"""Position encodings. Learned absolute positions: a table added to the token embedding
(damendaemon/gpt2.py:46); the add is fused into the embedding kernel. Rotary positions: queries and keys
are rotated in place, pair by pair, by position x frequency, before they are cached and attended; the
frequencies may be blended for a long context (``LongContextBlend``) or stretched by wavelength (``WavelengthStretch``)."""
from __future__ import annotations

import math

import torch

from .. import kernels
from .interfaces import PositionEncoding
from .registry import register_position
from .spec import TensorDecl, WavelengthStretch


@register_position("learned")
class LearnedPositions(PositionEncoding):
    def __init__(self, spec, weights, runtime):
        self.spec = spec
        self.table = weights[spec.table]

    @staticmethod
    def tensor_decls(spec):
        return [TensorDecl(spec.table, (spec.n_positions, spec.width), "table")]

    def embedding_table(self):
        return self.table


@register_position("none")
class NoPositions(PositionEncoding):
    def __init__(self, spec, weights, runtime):
        self.spec = spec


def rotary_frequencies(spec):
    """(float64 frequencies [dims/2], factor on cosine and sine). Plain: f_i = base^(-2i/dims). Stretched: see
    ``WavelengthStretch``. Blended: see
    ``LongContextBlend``; the pair that turns t times over the original length is
    dims * ln(original / (2 pi t)) / (2 ln base)."""
    half = spec.dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = float(spec.base) ** (-2.0 * i / spec.dims)
    b = spec.blend
    if b is None:
        return f, 1.0
    if isinstance(b, WavelengthStretch):
        length = 2 * math.pi / f
        s = (b.original / length - b.low) / (b.high - b.low)
        mixed = (1 - s) * f / b.factor + s * f
        f = torch.where(length < b.original / b.high, f, torch.where(length > b.original / b.low, f / b.factor, mixed))
        return f, 1.0
    pair_of = lambda turns: spec.dims * math.log(b.original / (2 * math.pi * turns)) / (2 * math.log(spec.base))
    lo = max(math.floor(pair_of(b.fast)), 0)
    hi = min(math.ceil(pair_of(b.slow)), spec.dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / b.factor * ramp + f * (1.0 - ramp), 0.1 * math.log(b.factor) + 1.0


@register_position("rotary")
class RotaryPositions(PositionEncoding):
    """Acts on queries and keys (``on_query_key``), as a model's position encoding or as a mixer's own."""

    def __init__(self, spec, weights, runtime):
        if spec.dims % 2 or not 0 < spec.dims <= spec.head_dim:
            raise ValueError(f"{spec.dims} rotated dimensions do not fit a head of {spec.head_dim} in pairs")
        self.spec = spec
        freqs, self.magnitude = rotary_frequencies(spec)
        self.freqs = freqs.to(torch.float32).to(runtime.device)

    def on_query_key(self, q, k, ctx):
        d = self.spec.head_dim
        return kernels.rotary(q, k, ctx.positions, self.freqs, self.magnitude, q.shape[1] // d, k.shape[1] // d, d,
                              self.spec.interleaved)
