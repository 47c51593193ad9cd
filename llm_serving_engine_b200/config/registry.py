"""One registry from an architecture's name to its configuration class and builder.

``config.json`` names its architecture in ``architectures[0]``; the reference
checks only ``model_type == "qwen2"`` (``src/llmserve/checkpoint.py:35-36``),
which is kept as the fallback when ``architectures`` is absent.
"""
from __future__ import annotations

import inspect
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .model_config import ConfigError, ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                      # has from_dict(dict)
    build_spec: Callable[[Any], ModelSpec]  # typed config -> ModelSpec
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class, build_spec, model_types=()) -> None:
    """Make ``name`` loadable.  ``config_class.from_dict`` parses config.json and
    ``build_spec`` turns the result into a ``ModelSpec``."""
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec, tuple(model_types))


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(values: dict[str, Any]) -> Architecture:
    names = values.get("architectures") or []
    if not names and isinstance(values.get("architecture"), str):   # some designs name theirs in one string
        names = [values["architecture"]]
    if names:
        entry = _ARCHITECTURES.get(names[0])
        if entry is None:
            raise ConfigError(f"unknown architecture {names[0]!r}; known: {known_architectures()}")
        return entry
    model_type = values.get("model_type")
    for entry in _ARCHITECTURES.values():
        if model_type in entry.model_types:
            return entry
    raise ConfigError(
        f"config.json names no architecture (architectures={names!r}, model_type={model_type!r}); "
        f"known: {known_architectures()}"
    )


def load_config(folder_or_dict) -> tuple[Architecture, Any, ModelSpec]:
    """Read config.json (or take its dictionary) and return the architecture
    entry, the typed configuration and the model description."""
    if isinstance(folder_or_dict, dict):
        values = folder_or_dict
    else:
        path = Path(folder_or_dict)
        if path.is_dir():
            path = path / "config.json"
        if not path.exists():
            raise ConfigError(f"no config.json at {path}")
        values = json.loads(path.read_text())
    entry = resolve_architecture(values)
    accepted = inspect.signature(entry.config_class.from_dict).parameters
    shapes = None
    if not isinstance(folder_or_dict, dict) and "tensor_shapes" in accepted:
        shapes = _checkpoint_tensor_shapes(Path(folder_or_dict))
    names = None if isinstance(folder_or_dict, dict) or shapes is not None else _checkpoint_tensor_names(Path(folder_or_dict))
    if shapes is not None:
        config = entry.config_class.from_dict(values, tensor_shapes=shapes)   # a design some of whose sizes only the tensors give
    elif names is not None and "tensor_names" in accepted:
        config = entry.config_class.from_dict(values, tensor_names=names)   # a design whose file leaves to the tensors what it has
    else:
        config = entry.config_class.from_dict(values)
    return entry, config, entry.build_spec(config)


def _checkpoint_tensor_shapes(folder: Path):
    """name -> shape of the tensors in the safetensors files beside config.json (None when there are none)."""
    folder = folder if folder.is_dir() else folder.parent
    files = sorted(folder.glob("*.safetensors"))
    if not files:
        return None
    from safetensors import safe_open

    shapes: dict[str, tuple] = {}
    for filename in files:
        with safe_open(str(filename), framework="pt", device="cpu") as source:
            for name in source.keys():
                shapes[name] = tuple(source.get_slice(name).get_shape())
    return shapes


def _checkpoint_tensor_names(folder: Path):
    """Names of the tensors in the safetensors files beside config.json (None when there are none)."""
    folder = folder if folder.is_dir() else folder.parent
    files = sorted(folder.glob("*.safetensors"))
    if not files:
        return None
    from safetensors import safe_open

    names: set[str] = set()
    for filename in files:
        with safe_open(str(filename), framework="pt", device="cpu") as source:
            names.update(source.keys())
    return frozenset(names)
