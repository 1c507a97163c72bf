"""Tetitar described with the framework's parts.

A decoder over a float32 stream that starts as the token's row plus a row of a hashed table of token pairs. A run of
layers may be repeated: every pass has caches and states of its own (a stop of the run order each), every pass after the
first starts by adding the embedding's output to the stream, and every pass by adding its row of a table of vectors. A
layer is pre-norm with norms that compute no statistics, tanh(alpha x) w + b. A mixer is one of
  attention   grouped attention over every earlier key whose values are the keys as projected; queries and keys normed
              over the whole projection, rotated (halves paired, frequencies stretched by wavelength), an element-wise
              sigmoid gate on the output;
  parallel    windowed attention (per-head norms, a unit term in the softmax's denominator) beside a state-space mixer,
              both outputs normed and averaged;
  rglru       a gated linear recurrence per channel behind a short convolution.
The feed-forward is a silu gated unit, or absent. The final norm, the token table as the head and a tanh cap give the logits.

Tensor names: embed, bigram, loop.step, l<i>.{norm1, norm2} each with .b and .alpha, l<i>.mix.* (attention: q, k, q.norm,
k.norm, g, o; parallel: left.{q, k, v, q.norm, k.norm, o, out}, right.{in, conv, conv.b, dt_bias, A_log, D, norm, o, out};
rglru: y, y.b, x, x.b, conv, conv.b, ra, ra.b, ri, ri.b, lam, o), l<i>.mlp.{gate, up, down}, final.norm (.b, .alpha);
matrices [out, in].
"""
from __future__ import annotations

import math

import torch

from ..config.tetitar import ARCHITECTURE, TetitarConfig
from ..parts.spec import (AttentionSpec, EmbeddingSpec, GatedFeedForwardSpec, GatedUnitSpec, HeadSpec, LayerSpec,
                          LinearRecurrenceSpec, ModelSpec, NoFeedForwardSpec, NormSpec, PairEmbeddingSpec, PositionSpec, RotarySpec,
                          RunEntry, SideBySideSpec, StateSpaceSpec, WavelengthStretch)
from ..registry import Architecture, register_architecture

RECURRENCE_GAIN = 8.0       # the design fixes the factor of the recurrence's decay, log a = -8 r softplus(lam)
BRANCH_FACTOR = 0.5         # and that the two mixers of a parallel layer are averaged


def _norm(c, name):
    return NormSpec("tanh", c.width, c.norm_eps, name, bias=name + ".b", alpha=name + ".alpha")


def _rotary(m):
    s = m.rot.scaling
    stretch = None if s is None else WavelengthStretch(s.factor, s.low, s.high, s.original)
    return RotarySpec("rotary", head_dim=m.dim, dims=m.rot.dims, base=m.rot.base, interleaved=False, blend=stretch)


def _mixer_spec(c: TetitarConfig, i: int):
    layer, p = c.layers[i], f"l{i}.mix."
    m = layer.mixer
    if layer.type == "attention":
        return AttentionSpec("attention", width=c.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
                             window=m.mask_size, qkv_weight=(p + "q", p + "k"), qkv_bias=None, out_weight=p + "o", out_bias=None,
                             value_dim=m.vdim, gate_weight=p + "g", rotary=_rotary(m), query_norm=p + "q.norm",
                             key_norm=p + "k.norm", head_norm_eps=c.norm_eps, values_are_keys=True, norm_whole_projection=True,
                             gate_per_element=True)
    if layer.type == "parallel":
        l, r = m.left, m.right
        left = AttentionSpec("attention", width=c.width, n_heads=l.heads, n_kv_heads=l.kv_heads, head_dim=l.dim, scale=l.scale,
                             window=l.mask_size, qkv_weight=(p + "left.q", p + "left.k", p + "left.v"), qkv_bias=None,
                             out_weight=p + "left.o", out_bias=None, value_dim=l.vdim, rotary=_rotary(l),
                             query_norm=p + "left.q.norm", key_norm=p + "left.k.norm", head_norm_eps=c.norm_eps, unit_sink=True)
        right = StateSpaceSpec("state_space", width=c.width, n_heads=r.heads, value_dim=r.vdim, state=r.state, groups=r.groups,
                               conv_taps=r.conv, norm_groups=r.norm_groups, norm_eps=c.norm_eps, in_weight=p + "right.in",
                               conv_weight=p + "right.conv", conv_bias=p + "right.conv.b", dt_bias=p + "right.dt_bias",
                               decay_log=p + "right.A_log", skip=p + "right.D", out_norm=p + "right.norm", out_weight=p + "right.o")
        return SideBySideSpec("side_by_side", width=c.width, left=left, right=right, left_norm=p + "left.out",
                              right_norm=p + "right.out", norm_eps=c.norm_eps, factor=BRANCH_FACTOR)
    return LinearRecurrenceSpec("linear_recurrence", width=c.width, inner=m.width, blocks=m.blocks, conv_taps=m.conv,
                                gain=RECURRENCE_GAIN, gate_weight=p + "y", gate_bias=p + "y.b", in_weight=p + "x", in_bias=p + "x.b",
                                conv_weight=p + "conv", conv_bias=p + "conv.b", decay_gate=p + "ra", decay_gate_bias=p + "ra.b",
                                input_gate=p + "ri", input_gate_bias=p + "ri.b", decay_param=p + "lam", out_weight=p + "o")


def _layer_spec(c: TetitarConfig, i: int):
    f, p = c.layers[i].mlp, f"l{i}."
    if f is None:
        return LayerSpec("pre_norm_mixer", _mixer_spec(c, i), NoFeedForwardSpec(), (_norm(c, p + "norm1"),))
    unit = GatedUnitSpec(f.ff, 0.0, p + "mlp.gate", p + "mlp.up", p + "mlp.down", activation="silu")
    return LayerSpec("pre_norm", _mixer_spec(c, i), GatedFeedForwardSpec("gated", c.width, unit),
                     (_norm(c, p + "norm1"), _norm(c, p + "norm2")))


def run_order(c: TetitarConfig):
    """The stops: layers before the loop once, the loop's layers ``times`` times (a pass's first stop adds its row of the
    pass vectors, and from the second pass on the embedding's output), then the rest."""
    n = len(c.layers)
    if c.loop is None:
        return tuple(RunEntry(i) for i in range(n))
    a, b = c.loop.start, c.loop.stop
    stops = [RunEntry(i) for i in range(a)]
    for t in range(c.loop.times):
        stops += [RunEntry(i, add_embedding=(t > 0 and i == a), add_vector=t if i == a else None) for i in range(a, b)]
    return tuple(stops + [RunEntry(i) for i in range(b, n)])


def build_spec(c: TetitarConfig) -> ModelSpec:
    if c.pairs is None:
        embedding = EmbeddingSpec("tokens", c.vocab, c.width, table="embed")
    else:
        embedding = PairEmbeddingSpec("tokens_pairs", c.vocab, c.width, table="embed", pair_table="bigram", buckets=c.pairs.buckets,
                                      mul_prev=c.pairs.mul_prev, mul_cur=c.pairs.mul_cur)
    looped = c.loop is not None and c.loop.stop > c.loop.start
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=c.vocab, width=c.width, max_positions=None, embedding=embedding,
        position=PositionSpec("none", 0, c.width), layers=tuple(_layer_spec(c, i) for i in range(len(c.layers))),
        run_order=run_order(c) if looped else tuple(RunEntry(i) for i in range(len(c.layers))),
        head=HeadSpec("linear", c.vocab, c.width, norm=_norm(c, "final.norm"), weight="embed", tied=True, softcap=c.logit_softcap),
        pass_vectors=("loop.step", c.loop.times) if looped else None,
        ignored_tensors=() if looped or c.loop is None else (r"loop\.step",), eos_token_ids=tuple(c.eos_token_ids))


def random_tensors(c: TetitarConfig, seed: int, matrix_dtype=torch.float32, device="cpu") -> dict:
    """Seeded random weights under their checkpoint names, in a fixed draw order: tables ~N(0, 1), matrices ~N(0, 1/in), norm
    weights ~N(1, 0.1), biases ~N(0, 0.1), alphas near 0.5, convolution taps ~N(0, 1/taps) with the current token's tap near
    one, decay parameters spread so that fast and slow channels and heads both occur."""
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    out = {}
    normal = lambda *shape: torch.randn(shape, generator=g, dtype=torch.float32, device=device)

    def matrix(name, rows, cols, gain=1.0):
        out[name] = (normal(rows, cols) * gain / math.sqrt(cols)).to(matrix_dtype)

    def around(name, n, centre=1.0, spread=0.1):
        out[name] = centre + normal(n) * spread

    def norm(name):
        around(name, c.width)
        around(name + ".b", c.width, centre=0.0)
        out[name + ".alpha"] = 0.5 + 0.1 * normal()

    def conv(name, channels, taps):
        w = normal(channels, taps) / math.sqrt(taps)
        w[:, -1] += 1.0
        out[name] = w
        around(name + ".b", channels, centre=0.0)

    def attention(p, m, own_values):
        matrix(p + "q", m.heads * m.dim, c.width)
        matrix(p + "k", m.kv_heads * m.dim, c.width)
        if own_values:
            matrix(p + "v", m.kv_heads * m.vdim, c.width)
            around(p + "q.norm", m.dim)
            around(p + "k.norm", m.dim)
        else:
            around(p + "q.norm", m.heads * m.dim)
            around(p + "k.norm", m.kv_heads * m.dim)
            matrix(p + "g", m.heads * m.vdim, c.width)
        matrix(p + "o", c.width, m.heads * m.vdim)

    out["embed"] = normal(c.vocab, c.width).to(matrix_dtype)
    if c.pairs is not None:
        out["bigram"] = (normal(c.pairs.buckets + 1, c.width) * 0.5).to(matrix_dtype)
    if c.loop is not None:
        out["loop.step"] = normal(c.loop.times, c.width) * 0.3
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        norm(p + "norm1")
        if layer.type == "attention":
            attention(p + "mix.", m, False)
        elif layer.type == "parallel":
            attention(p + "mix.left.", m.left, True)
            r, q = m.right, p + "mix.right."
            inner = r.heads * r.vdim
            matrix(q + "in", 2 * inner + 2 * r.groups * r.state + r.heads, c.width)
            conv(q + "conv", inner + 2 * r.groups * r.state, r.conv)
            around(q + "dt_bias", r.heads, centre=-1.0, spread=1.0)
            out[q + "A_log"] = normal(r.heads) * 0.7 - 0.5
            around(q + "D", r.heads)
            around(q + "norm", inner)
            matrix(q + "o", c.width, inner)
            around(p + "mix.left.out", c.width)
            around(p + "mix.right.out", c.width)
        else:
            part = m.width // m.blocks
            matrix(p + "mix.y", m.width, c.width)
            around(p + "mix.y.b", m.width, centre=0.0)
            matrix(p + "mix.x", m.width, c.width)
            around(p + "mix.x.b", m.width, centre=0.0)
            conv(p + "mix.conv", m.width, m.conv)
            for name in ("ra", "ri"):
                out[p + "mix." + name] = normal(m.blocks, part, part) / math.sqrt(part)
                out[p + "mix." + name + ".b"] = normal(m.blocks, part) * 0.1
            out[p + "mix.lam"] = normal(m.width) * 1.5 - 2.0
            matrix(p + "mix.o", c.width, m.width)
        if layer.mlp is not None:
            norm(p + "norm2")
            matrix(p + "mlp.gate", layer.mlp.ff, c.width)
            matrix(p + "mlp.up", layer.mlp.ff, c.width)
            matrix(p + "mlp.down", c.width, layer.mlp.ff)
    norm("final.norm")
    return out


register_architecture(Architecture(ARCHITECTURE, TetitarConfig.from_dict, build_spec, random_tensors), replace=True)
