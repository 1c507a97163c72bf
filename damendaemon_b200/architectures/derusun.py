"""Derusun described with the framework's parts.

A decoder over a float32 stream that starts as the token's row. Every layer is pre-norm: x <- x + mixer(shift(norm1(x))),
then, where the layer has one, x <- x + ff(norm2(x)). The norms divide each of ``groups`` equal stretches of the row by its
own root mean square; the shift blends a normed row, per channel, with the normed row of the token before. What a layer
hands on is not its own result alone but a learned weighted sum of the embedding's output and every layer's result so far
(``ModelSpec.depth_mix``). A mixer is one of
  channel_delta     the gated delta rule with a decay per key channel (short convolutions, unit q and k, low-rank decay
                    and output gate, a per-request float32 state);
  latent_attention  attention whose keys and values are projections of one cached latent row per token, with a rotated
                    key part that all heads share and a sink in the softmax;
  attention         grouped attention with projection biases, per-head norms of q and k, no positions, capped scores, a
                    window that keeps the sequence's first keys visible, a sink, and values blended with those of the
                    first such layer.
The feed-forward is a clamped gated unit. The final norm (in groups as well) and an untied head give the logits.

Tensor names: embed, l<i>.{norm1, norm2, shift, dwa}, l<i>.mix.* (channel_delta: q, k, v each with .conv, b, A_log, a1,
a2, dt_bias, g1, g2, norm, o; latent_attention: q, dkv, dkv.norm, uk, uv, sink, o; attention: q, k, v each with .b,
q.norm, k.norm, sink, vmix, o), l<i>.mlp.{gate, up, down}, final.norm, head; matrices [out, in].
"""
from __future__ import annotations

import math

import torch

from ..config.derusun import ARCHITECTURE, DerusunConfig
from ..parts.spec import (AttentionSpec, EmbeddingSpec, GatedDeltaSpec, GatedFeedForwardSpec, GatedUnitSpec, HeadSpec,
                          LatentAttentionSpec, LayerSpec, ModelSpec, NoFeedForwardSpec, NormSpec, PositionSpec, RotarySpec,
                          RunEntry)
from ..registry import Architecture, register_architecture

SWISH_ALPHA = 1.702       # the design fixes the sigmoid's slope in its gated unit


def _norm(c, name):
    return NormSpec("rmsnorm", c.width, c.norm_eps, name, groups=c.norm_groups)


def _first_mixing_layer(c: DerusunConfig):
    return next((i for i, l in enumerate(c.layers) if l.type == "attention" and l.mixer.v_mix), None)


def _mixer_spec(c: DerusunConfig, i: int):
    layer, p = c.layers[i], f"l{i}.mix."
    m = layer.mixer
    if layer.type == "channel_delta":
        if m.decay_rank is None or m.gate_rank is None:
            raise ValueError(f"layer {i}: the ranks of the gated-delta mixer's low-rank projections are not known; read them "
                             "from the tensors' shapes (DerusunConfig.with_tensor_shapes) or name them")
        return GatedDeltaSpec("gated_delta", width=c.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                              value_dim=m.vdim, conv_taps=m.conv, decay_rank=m.decay_rank, gate_rank=m.gate_rank,
                              norm_eps=c.norm_eps, query_weight=p + "q", key_weight=p + "k", value_weight=p + "v",
                              beta_weight=p + "b", decay_down=p + "a1", decay_up=p + "a2", decay_log=p + "A_log",
                              decay_bias=p + "dt_bias", gate_down=p + "g1", gate_up=p + "g2", out_norm=p + "norm",
                              out_weight=p + "o")
    if layer.type == "latent_attention":
        return LatentAttentionSpec("latent_attention", width=c.width, n_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim,
                                   value_dim=m.vdim, rank=m.kv_rank, scale=m.scale, norm_eps=c.norm_eps,
                                   rotary=RotarySpec("rotary", head_dim=m.rot_dim, dims=m.rot_dims, base=m.rot_base, interleaved=True),
                                   query_weight=p + "q", down_weight=p + "dkv", latent_norm=p + "dkv.norm",
                                   up_key_weight=p + "uk", up_value_weight=p + "uv", out_weight=p + "o", sink=p + "sink")
    first = _first_mixing_layer(c)
    return AttentionSpec("attention", width=c.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
                         window=m.mask_size, qkv_weight=(p + "q", p + "k", p + "v"), qkv_bias=(p + "q.b", p + "k.b", p + "v.b"),
                         out_weight=p + "o", out_bias=None, value_dim=m.vdim, query_norm=p + "q.norm", key_norm=p + "k.norm",
                         head_norm_eps=c.norm_eps, keep_first=m.keep_first if m.mask_size is not None else 0,
                         softcap=m.softcap, sink=p + "sink", value_mix_source=m.v_mix and first == i,
                         value_mix=p + "vmix" if m.v_mix and first != i else None, exact_weights=True)


def _layer_spec(c: DerusunConfig, i: int):
    f, p = c.layers[i].mlp, f"l{i}."
    if f is None:
        return LayerSpec("pre_norm_shift", _mixer_spec(c, i), NoFeedForwardSpec(), (_norm(c, p + "norm1"),), shift_weight=p + "shift")
    unit = GatedUnitSpec(f.ff, f.limit, p + "mlp.gate", p + "mlp.up", p + "mlp.down", alpha=SWISH_ALPHA, activation="clamped_swish")
    return LayerSpec("pre_norm_shift", _mixer_spec(c, i), GatedFeedForwardSpec("gated", c.width, unit),
                     (_norm(c, p + "norm1"), _norm(c, p + "norm2")), shift_weight=p + "shift")


def build_spec(c: DerusunConfig) -> ModelSpec:
    n = len(c.layers)
    first = _first_mixing_layer(c)
    # every layer that blends values has a weight for it; the first such layer's blends with nothing and is not read (nor
    # would be one stored with an attention layer that does not blend)
    unused = tuple(rf"l{i}\.mix\.vmix" for i, l in enumerate(c.layers) if l.type == "attention" and (not l.mixer.v_mix or i == first))
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=c.vocab, width=c.width, max_positions=None,
        embedding=EmbeddingSpec("tokens", c.vocab, c.width, table="embed"),
        position=PositionSpec("none", 0, c.width), layers=tuple(_layer_spec(c, i) for i in range(n)),
        run_order=tuple(RunEntry(i) for i in range(n)),
        head=HeadSpec("linear", c.vocab, c.width, norm=_norm(c, "final.norm"), weight="head"),
        depth_mix=tuple(f"l{i}.dwa" for i in range(n)), eos_token_ids=tuple(c.eos_token_ids), ignored_tensors=unused)


def with_tensor_shapes(c: DerusunConfig, shapes: dict) -> DerusunConfig:
    return c.with_tensor_shapes(shapes)


def random_tensors(c: DerusunConfig, seed: int, matrix_dtype=torch.float32, device="cpu") -> dict:
    """Seeded random weights under their checkpoint names, in a fixed draw order: the token table ~N(0, 1), matrices
    ~N(0, 1/in), norm weights ~N(1, 0.1), biases ~N(0, 0.1), shift weights uniform in [0, 1], convolution taps ~N(0, 1/taps)
    with the current token's tap near one, depth weights that favour the newest stream. A gated-delta layer whose ranks the
    configuration does not name gets ranks of half its key size (at least 8)."""
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    out = {}
    normal = lambda *shape: torch.randn(shape, generator=g, dtype=torch.float32, device=device)

    def matrix(name, rows, cols, gain=1.0):
        out[name] = (normal(rows, cols) * gain / math.sqrt(cols)).to(matrix_dtype)

    def around(name, n, centre=1.0, spread=0.1):
        out[name] = centre + normal(n) * spread

    out["embed"] = normal(c.vocab, c.width).to(matrix_dtype)
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        around(p + "norm1", c.width)
        out[p + "shift"] = torch.rand((c.width,), generator=g, dtype=torch.float32, device=device)
        if layer.type == "channel_delta":
            qk, v = m.kv_heads * m.dim, m.heads * m.vdim
            decay_rank = m.decay_rank or max(8, m.dim // 2)
            gate_rank = m.gate_rank or max(8, m.dim // 2)
            for name, rows in (("q", qk), ("k", qk), ("v", v)):
                matrix(p + "mix." + name, rows, c.width)
                taps = normal(rows, m.conv) / math.sqrt(m.conv)
                taps[:, -1] += 1.0
                out[p + "mix." + name + ".conv"] = taps
            matrix(p + "mix.b", m.heads, c.width)
            out[p + "mix.A_log"] = normal(m.heads) * 0.5 - 1.0
            around(p + "mix.norm", m.vdim)
            matrix(p + "mix.a1", decay_rank, c.width)
            matrix(p + "mix.a2", m.heads * m.dim, decay_rank)
            around(p + "mix.dt_bias", m.heads * m.dim, centre=-1.0, spread=1.0)
            matrix(p + "mix.g1", gate_rank, c.width)
            matrix(p + "mix.g2", v, gate_rank)
            matrix(p + "mix.o", c.width, v)
        elif layer.type == "latent_attention":
            matrix(p + "mix.q", m.heads * (m.dim + m.rot_dim), c.width)
            matrix(p + "mix.dkv", m.kv_rank + m.rot_dim, c.width)
            around(p + "mix.dkv.norm", m.kv_rank)
            matrix(p + "mix.uk", m.heads * m.dim, m.kv_rank)
            matrix(p + "mix.uv", m.heads * m.vdim, m.kv_rank)
            around(p + "mix.sink", m.heads, centre=0.0, spread=1.0)
            matrix(p + "mix.o", c.width, m.heads * m.vdim)
        else:
            for name, rows in (("q", m.heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim)):
                matrix(p + "mix." + name, rows, c.width)
                around(p + "mix." + name + ".b", rows, centre=0.0)
            around(p + "mix.q.norm", m.dim)
            around(p + "mix.k.norm", m.dim)
            around(p + "mix.sink", m.heads, centre=0.0, spread=1.0)
            if m.v_mix:
                out[p + "mix.vmix"] = torch.rand((), generator=g, dtype=torch.float32, device=device)
            matrix(p + "mix.o", c.width, m.heads * m.vdim)
        if layer.mlp is not None:
            around(p + "norm2", c.width)
            matrix(p + "mlp.gate", layer.mlp.ff, c.width)
            matrix(p + "mlp.up", layer.mlp.ff, c.width)
            matrix(p + "mlp.down", c.width, layer.mlp.ff)
        mix = normal(i + 2) * 0.2
        mix[-1] += 1.0
        out[p + "dwa"] = mix
    around("final.norm", c.width)
    matrix("head", c.vocab, c.width)
    return out


register_architecture(Architecture(ARCHITECTURE, DerusunConfig.from_dict, build_spec, random_tensors,
                                   sizes_from_shapes=with_tensor_shapes), replace=True)
