"""The one registry from an architecture's name to its configuration and model.

``config.json``'s ``architectures[0]`` (or its ``architecture``, where a model names one so) selects the entry everywhere in the framework
(engine, command line, trace replay, random-weights writer). The reference
dispatches on ``model_type`` in three places (damendaemon/config.py:119-145,
damendaemon/runtime.py:675-679, damendaemon/qwen2.py:195-196); here it is one table.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .config.reader import ConfigError, read_config_file


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable      # dict -> typed config
    build_spec: Callable        # typed config -> ModelSpec
    random_tensors: Callable    # (typed config, seed, matrix dtype) -> {checkpoint name: tensor}
    # (typed config, {checkpoint name: shape}) -> typed config: for an architecture whose config.json leaves sizes to the
    # tensors' shapes; None where config.json says everything
    sizes_from_shapes: Callable = None


ARCHITECTURES: dict = {}


def register_architecture(entry: Architecture, *, replace=False):
    if entry.name in ARCHITECTURES and not replace:
        raise ValueError(f"architecture {entry.name!r} is already registered")
    ARCHITECTURES[entry.name] = entry
    return entry


def architecture_of(config: dict) -> Architecture:
    names = config.get("architectures")
    if names is None and isinstance(config.get("architecture"), str):
        names = [config["architecture"]]
    if not isinstance(names, list) or len(names) != 1 or not isinstance(names[0], str):
        raise ConfigError(f"config.json 'architectures' must name exactly one architecture, got {names!r}")
    _load_builtin()
    if names[0] not in ARCHITECTURES:
        raise ConfigError(f"unknown architecture {names[0]!r}; known: {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[names[0]]


def load_config(model_dir):
    """Folder -> (Architecture, typed config); sizes that only the tensors' shapes give are read from the weight files'
    headers."""
    raw = read_config_file(model_dir)
    arch = architecture_of(raw)
    typed = arch.parse_config(raw)
    if arch.sizes_from_shapes is not None:
        from .weights.loader import tensor_shapes
        typed = arch.sizes_from_shapes(typed, tensor_shapes(model_dir))
    return arch, typed


def _load_builtin():
    from .architectures import bonatar, derusun, gpt2, tetitar, zokanex  # noqa: F401  (register themselves on import)
