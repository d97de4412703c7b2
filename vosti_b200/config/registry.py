"""One registry from an architecture's name to the function that turns its
config.json into a `ModelSpec`.

The reference dispatches on a closed enum (src/model_config.rs:11-16,
src/exec/model.rs:205-621) keyed by its own family name; here the key is
``config.json: architectures[0]`` and the table is open.
"""
from __future__ import annotations

import inspect
import json
from pathlib import Path
from typing import Any, Callable, Dict, Mapping, Optional

from .schema import ConfigError, ModelSpec

_ARCHITECTURES: Dict[str, Callable[[Mapping[str, Any]], ModelSpec]] = {}


def register_architecture(name: str, spec_from_config: Callable[[Mapping[str, Any]], ModelSpec],
                          *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = spec_from_config


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(raw: Mapping[str, Any]) -> str:
    """The name a config.json gives its design: the one entry of 'architectures', or the
    string 'architecture' for families that write it so."""
    names = raw.get("architectures") if isinstance(raw, Mapping) else None
    if names is None and isinstance(raw, Mapping) and isinstance(raw.get("architecture"), str):
        return raw["architecture"]
    if not isinstance(names, list) or len(names) != 1 or not isinstance(names[0], str):
        raise ConfigError("config.json must name exactly one architecture in 'architectures' (or 'architecture')")
    return names[0]


def _wants_shapes(fn: Callable) -> bool:
    try:
        return "shapes" in inspect.signature(fn).parameters
    except (TypeError, ValueError):
        return False


def model_spec_from_config(raw: Mapping[str, Any], shapes: Optional[Mapping[str, tuple]] = None) -> ModelSpec:
    """`shapes` (tensor name -> shape) is handed to architectures whose config.json leaves some
    sizes to the checkpoint's tensor shapes; their function takes a `shapes` argument."""
    name = architecture_of(raw)
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{name}'; known: {known_architectures()}")
    fn = _ARCHITECTURES[name]
    spec = fn(raw, shapes=shapes) if _wants_shapes(fn) else fn(raw)
    spec.validate()
    return spec


def read_config_json(model_dir: str | Path) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path} is not valid JSON: {error}") from error


def model_spec_from_dir(model_dir: str | Path) -> ModelSpec:
    raw = read_config_json(model_dir)
    shapes = None
    if _wants_shapes(_ARCHITECTURES.get(architecture_of(raw), lambda raw: None)):
        from ..weights.safetensors_io import open_model_shards
        shards = open_model_shards(model_dir)
        shapes = {name: tuple(shard.info(name)[1]) for name, shard in shards.items()}
    return model_spec_from_config(raw, shapes)
