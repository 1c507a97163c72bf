"""Typed Derusun configuration, parsed from the architecture's own config.json keys.

    architecture   "Derusun"
    vocab, width   sizes of the token table and the residual stream
    norm           {eps, groups}: of the layers' norms and the final one (a row in `groups` equal stretches, each divided
                   by its own root mean square); eps also serves the norms inside the mixers
    layers         a list; each entry {type, mixer: {...}, mlp: {kind: "dense", ff, limit} | null}
      channel_delta     {heads, kv_heads, dim, vdim, conv}: the gated delta rule with a decay per key channel; the ranks of
                        its two low-rank projections are not in config.json: the tensors' shapes give them
                        (``with_tensor_shapes``); a configuration that is to be filled with random weights may name them
                        (decay_rank, gate_rank)
      latent_attention  {heads, dim, rot_dim, vdim, kv_rank, scale, rot: {dims, base}}
      attention         {heads, kv_heads, dim, vdim, scale, softcap (optional), mask: {size, keep_first} (optional),
                        v_mix (optional)}

The configuration names no context length: the engine's cache sets it.
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass
from typing import Optional, Tuple

from .reader import ConfigError

ARCHITECTURE = "Derusun"


def _get(config, name, where):
    if not isinstance(config, dict) or name not in config:
        raise ConfigError(f"{where}: '{name}' is missing")
    return config[name]


def _positive_int(config, name, where):
    value = _get(config, name, where)
    if type(value) is not int or value <= 0:
        raise ConfigError(f"{where}.{name} must be a positive integer, got {value!r}")
    return value


def _number(config, name, where, positive=True):
    value = _get(config, name, where)
    if type(value) not in (int, float) or not math.isfinite(value) or (positive and value <= 0):
        raise ConfigError(f"{where}.{name} must be a finite{' positive' if positive else ''} number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int] = None      # from the tensors' shapes (or named, for random weights)
    gate_rank: Optional[int] = None


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float] = None
    mask_size: Optional[int] = None
    keep_first: int = 0
    v_mix: bool = False


@dataclass(frozen=True)
class Mlp:
    kind: str            # 'dense'
    ff: int
    limit: float


@dataclass(frozen=True)
class Layer:
    type: str            # 'channel_delta' | 'latent_attention' | 'attention'
    mixer: object
    mlp: Optional[Mlp]


def _shared_heads(sizes, where):
    if sizes["heads"] % sizes["kv_heads"]:
        raise ConfigError(f"{where}: {sizes['heads']} heads cannot share {sizes['kv_heads']} key heads")


def _delta(raw, where):
    sizes = {n: _positive_int(raw, n, where) for n in ("heads", "kv_heads", "dim", "vdim", "conv")}
    _shared_heads(sizes, where)
    ranks = {n: _positive_int(raw, n, where) for n in ("decay_rank", "gate_rank") if isinstance(raw, dict) and raw.get(n) is not None}
    return DeltaMixer(**sizes, **ranks)


def _latent(raw, where):
    sizes = {n: _positive_int(raw, n, where) for n in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
    rot = _get(raw, "rot", where)
    dims = _positive_int(rot, "dims", where + ".rot")
    if dims % 2 or dims > sizes["rot_dim"]:
        raise ConfigError(f"{where}.rot.dims must be even and at most rot_dim, got {dims}")
    base = _number(rot, "base", where + ".rot")
    if base == 1.0:
        raise ConfigError(f"{where}.rot.base must not be 1")
    return LatentMixer(scale=_number(raw, "scale", where), rot_dims=dims, rot_base=base, **sizes)


def _attention(raw, where):
    sizes = {n: _positive_int(raw, n, where) for n in ("heads", "kv_heads", "dim", "vdim")}
    _shared_heads(sizes, where)
    mask = raw.get("mask")
    size, keep = None, 0
    if mask is not None:
        size = _positive_int(mask, "size", where + ".mask")
        keep = mask.get("keep_first", 0)
        if type(keep) is not int or keep < 0:
            raise ConfigError(f"{where}.mask.keep_first must be a non-negative integer, got {keep!r}")
    cap = raw.get("softcap")
    if cap is not None:
        cap = _number(raw, "softcap", where)
    v_mix = raw.get("v_mix", False)
    if type(v_mix) is not bool:
        raise ConfigError(f"{where}.v_mix must be true or false, got {v_mix!r}")
    return AttentionMixer(scale=_number(raw, "scale", where), softcap=cap, mask_size=size, keep_first=keep, v_mix=v_mix, **sizes)


def _mlp(raw, where):
    if raw is None:
        return None
    kind = _get(raw, "kind", where)
    if kind != "dense":
        raise ConfigError(f"{where}.kind must be 'dense', got {kind!r}")
    return Mlp("dense", ff=_positive_int(raw, "ff", where), limit=_number(raw, "limit", where))


_MIXERS = {"channel_delta": _delta, "latent_attention": _latent, "attention": _attention}


@dataclass(frozen=True)
class DerusunConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    layers: Tuple[Layer, ...]
    eos_token_ids: tuple = ()

    architecture = ARCHITECTURE

    @property
    def vocab_size(self):
        return self.vocab

    @classmethod
    def from_dict(cls, config: dict) -> "DerusunConfig":
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
        mixing = [l.mixer for l in layers if l.type == "attention" and l.mixer.v_mix]
        if any((m.kv_heads, m.vdim) != (mixing[0].kv_heads, mixing[0].vdim) for m in mixing):
            raise ConfigError("layers that blend their values with the first such layer's must have its value heads and size")
        norm = _get(config, "norm", "config")
        width, groups = _positive_int(config, "width", "config"), _positive_int(norm, "groups", "norm")
        if width % groups:
            raise ConfigError(f"norm.groups: a row of {width} does not fall into {groups} equal stretches")
        return cls(vocab=_positive_int(config, "vocab", "config"), width=width, norm_eps=_number(norm, "eps", "norm"),
                   norm_groups=groups, layers=tuple(layers))

    def with_tensor_shapes(self, shapes: dict) -> "DerusunConfig":
        """The sizes that config.json does not name, from the checkpoint's tensor shapes ({name: shape}): the ranks of a
        gated-delta layer's low-rank projections, rows of 'l<i>.mix.a1' and 'l<i>.mix.g1'."""
        layers = []
        for i, layer in enumerate(self.layers):
            if layer.type == "channel_delta":
                found = {}
                for field, name in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                    shape = shapes.get(name)
                    named = getattr(layer.mixer, field)
                    if shape is not None and len(shape) == 2:
                        if named is not None and named != shape[0]:
                            raise ConfigError(f"layers[{i}].mixer.{field} is {named}, but {name} has {shape[0]} rows")
                        found[field] = int(shape[0])
                    elif named is None:
                        raise ConfigError(f"layers[{i}]: neither config.json nor a tensor {name} gives the mixer's {field}")
                layer = dataclasses.replace(layer, mixer=dataclasses.replace(layer.mixer, **found))
            layers.append(layer)
        return dataclasses.replace(self, layers=tuple(layers))

    def to_dict(self) -> dict:
        """The config.json this configuration round-trips through."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "channel_delta":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
                for field in ("decay_rank", "gate_rank"):
                    if getattr(m, field) is not None:
                        mixer[field] = getattr(m, field)
            elif layer.type == "latent_attention":
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                         "scale": m.scale, "rot": {"dims": m.rot_dims, "base": m.rot_base}}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.softcap is not None:
                    mixer["softcap"] = m.softcap
                if m.mask_size is not None:
                    mixer["mask"] = {"size": m.mask_size, "keep_first": m.keep_first}
                if m.v_mix:
                    mixer["v_mix"] = True
            mlp = None if layer.mlp is None else {"kind": "dense", "ff": layer.mlp.ff, "limit": layer.mlp.limit}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "layers": layers}
