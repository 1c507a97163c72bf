"""Typed Tetitar configuration, parsed from the architecture's own config.json keys.

    architecture   "Tetitar"
    vocab, width   sizes of the token table and the residual stream
    embedding      {bigram: {buckets, mul_prev, mul_cur}}: the table of token pairs that is added to the token's row
    norm           {eps}: of the norms inside the mixers (the layers' own norms compute no statistics)
    loop           {start, stop, times} (optional): layers start .. stop - 1 run `times` times in a row
    logit_softcap  c (optional): logits become c * tanh(logits / c)
    layers         a list; each entry {type, mixer: {...}, mlp: {kind: "dense", ff} | null}
      attention    {heads, kv_heads, dim, vdim, scale, rot: {dims, base, scaling (optional): {factor, low, high, original}},
                   mask (optional): {size}}: values are the keys as projected
      parallel     {left: an attention with values of its own, {heads, kv_heads, dim, vdim, scale, rot, mask (optional)},
                    right: {heads, vdim, state, groups, conv, norm_groups}, a state-space mixer}
      rglru        {width, blocks, conv}: a gated linear recurrence per channel

The configuration names no context length: the engine's cache sets it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

from .reader import ConfigError

ARCHITECTURE = "Tetitar"


def _get(config, name, where):
    if not isinstance(config, dict) or name not in config:
        raise ConfigError(f"{where}: '{name}' is missing")
    return config[name]


def _int(config, name, where, least=1):
    value = _get(config, name, where)
    if type(value) is not int or value < least:
        raise ConfigError(f"{where}.{name} must be an integer of at least {least}, got {value!r}")
    return value


def _number(config, name, where, positive=True):
    value = _get(config, name, where)
    if type(value) not in (int, float) or not math.isfinite(value) or (positive and value <= 0):
        raise ConfigError(f"{where}.{name} must be a finite{' positive' if positive else ''} number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class Stretch:
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    scaling: Optional[Stretch] = None


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotation
    mask_size: Optional[int] = None


@dataclass(frozen=True)
class StateSpaceMixer:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class ParallelMixer:
    left: AttentionMixer
    right: StateSpaceMixer


@dataclass(frozen=True)
class RecurrenceMixer:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class Mlp:
    kind: str            # 'dense'
    ff: int


@dataclass(frozen=True)
class Layer:
    type: str            # 'attention' | 'parallel' | 'rglru'
    mixer: object
    mlp: Optional[Mlp]


@dataclass(frozen=True)
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


def _rotation(raw, dim, where):
    dims = _int(raw, "dims", where)
    if dims % 2 or dims > dim:
        raise ConfigError(f"{where}.dims must be even and at most the head size {dim}, got {dims}")
    base = _number(raw, "base", where)
    if base == 1.0:
        raise ConfigError(f"{where}.base must not be 1")
    scaling = raw.get("scaling")
    if scaling is not None:
        scaling = Stretch(*(_number(scaling, n, where + ".scaling") for n in ("factor", "low", "high", "original")))
        if scaling.high == scaling.low:
            raise ConfigError(f"{where}.scaling: low and high must differ")
    return Rotation(dims, base, scaling)


def _attention(raw, where, own_values):
    sizes = {n: _int(raw, n, where) for n in ("heads", "kv_heads", "dim", "vdim")}
    if sizes["heads"] % sizes["kv_heads"]:
        raise ConfigError(f"{where}: {sizes['heads']} heads cannot share {sizes['kv_heads']} key heads")
    if not own_values and sizes["vdim"] != sizes["dim"]:
        raise ConfigError(f"{where}: values that are the keys have the keys' size, got dim {sizes['dim']} and vdim {sizes['vdim']}")
    mask = raw.get("mask")
    return AttentionMixer(scale=_number(raw, "scale", where), rot=_rotation(_get(raw, "rot", where), sizes["dim"], where + ".rot"),
                          mask_size=None if mask is None else _int(mask, "size", where + ".mask"), **sizes)


def _state_space(raw, where):
    m = StateSpaceMixer(**{n: _int(raw, n, where) for n in ("heads", "vdim", "state", "groups", "conv", "norm_groups")})
    if m.heads % m.groups:
        raise ConfigError(f"{where}: {m.heads} heads cannot share {m.groups} groups")
    if (m.heads * m.vdim) % m.norm_groups:
        raise ConfigError(f"{where}: {m.heads * m.vdim} channels do not fall into {m.norm_groups} equal parts")
    return m


def _parallel(raw, where):
    return ParallelMixer(_attention(_get(raw, "left", where), where + ".left", True), _state_space(_get(raw, "right", where), where + ".right"))


def _recurrence(raw, where):
    m = RecurrenceMixer(**{n: _int(raw, n, where) for n in ("width", "blocks", "conv")})
    if m.width % m.blocks:
        raise ConfigError(f"{where}: {m.width} channels do not fall into {m.blocks} equal parts")
    return m


def _mlp(raw, where):
    if raw is None:
        return None
    kind = _get(raw, "kind", where)
    if kind != "dense":
        raise ConfigError(f"{where}.kind must be 'dense', got {kind!r}")
    return Mlp("dense", ff=_int(raw, "ff", where))


_MIXERS = {"attention": lambda raw, where: _attention(raw, where, False), "parallel": _parallel, "rglru": _recurrence}


@dataclass(frozen=True)
class TetitarConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Layer, ...]
    pairs: Optional[PairTable] = None
    loop: Optional[Loop] = None
    logit_softcap: Optional[float] = None
    eos_token_ids: tuple = ()

    architecture = ARCHITECTURE

    @property
    def vocab_size(self):
        return self.vocab

    @classmethod
    def from_dict(cls, config: dict) -> "TetitarConfig":
        if config.get("architecture") != ARCHITECTURE:
            raise ConfigError(f"architecture must be {ARCHITECTURE!r}, got {config.get('architecture')!r}")
        raw_layers = _get(config, "layers", "config")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, raw in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _get(raw, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}.type must be one of {sorted(_MIXERS)}, got {kind!r}")
            layers.append(Layer(kind, _MIXERS[kind](_get(raw, "mixer", where), where + ".mixer"), _mlp(raw.get("mlp"), where + ".mlp")))
        pairs = (config.get("embedding") or {}).get("bigram")
        if pairs is not None:
            pairs = PairTable(_int(pairs, "buckets", "embedding.bigram"), _int(pairs, "mul_prev", "embedding.bigram", 0),
                              _int(pairs, "mul_cur", "embedding.bigram", 0))
        loop = config.get("loop")
        if loop is not None:
            loop = Loop(_int(loop, "start", "loop", 0), _int(loop, "stop", "loop", 0), _int(loop, "times", "loop"))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"loop: layers {loop.start} to {loop.stop} are not a run of the model's {len(layers)} layers")
        cap = config.get("logit_softcap")
        if cap is not None:
            cap = _number(config, "logit_softcap", "config")
        return cls(vocab=_int(config, "vocab", "config"), width=_int(config, "width", "config"),
                   norm_eps=_number(_get(config, "norm", "config"), "eps", "norm"), layers=tuple(layers), pairs=pairs, loop=loop,
                   logit_softcap=cap)

    def to_dict(self) -> dict:
        """The config.json this configuration round-trips through."""
        def rot(r):
            out = {"dims": r.dims, "base": r.base}
            if r.scaling is not None:
                s = r.scaling
                out["scaling"] = {"factor": s.factor, "low": s.low, "high": s.high, "original": s.original}
            return out

        def attention(m):
            out = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "rot": rot(m.rot)}
            if m.mask_size is not None:
                out["mask"] = {"size": m.mask_size}
            return out

        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                mixer = attention(m)
            elif layer.type == "parallel":
                r = m.right
                mixer = {"left": attention(m.left),
                         "right": {"heads": r.heads, "vdim": r.vdim, "state": r.state, "groups": r.groups, "conv": r.conv,
                                   "norm_groups": r.norm_groups}}
            else:
                mixer = {"width": m.width, "blocks": m.blocks, "conv": m.conv}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": None if layer.mlp is None else {"kind": "dense", "ff": layer.mlp.ff}})
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.pairs is not None:
            out["embedding"] = {"bigram": {"buckets": self.pairs.buckets, "mul_prev": self.pairs.mul_prev, "mul_cur": self.pairs.mul_cur}}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out
