"""The one registry from an architecture's name to its model.

An entry holds two functions: ``read_config(dict) -> typed config`` and
``model_spec(config) -> ModelSpec``.  The role of snowllm/models/__init__.py:9-38
(architecture string -> module, error lists what is supported).
"""
from __future__ import annotations

import json
import pathlib
from dataclasses import dataclass
from typing import Any, Callable

from ..errors import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable[[dict], Any]
    model_spec: Callable[[Any], Any]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, read_config, model_spec) -> None:
    """Make ``name`` (as config.json's ``architectures`` spells it) loadable."""
    _ARCHITECTURES[name] = Architecture(name, read_config, model_spec)


def architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def resolve(names) -> Architecture:
    """First registered name among config.json's ``architectures``."""
    _load_builtin()
    for n in names or ():
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    raise ConfigError(f"no supported architecture among {list(names or ())!r}; "
                      f"supported: {', '.join(sorted(_ARCHITECTURES))}")


def _load_builtin() -> None:
    from ..models import lfm2  # noqa: F401  (registers itself on import)


def read_config_json(path) -> tuple[Architecture, Any, dict]:
    """(architecture entry, typed config, raw dict) of a model folder's config.json.
    ``text_config`` is taken where present; ``architectures`` may sit on either level
    (snowllm/checkpoint/loader.py:203-207)."""
    path = pathlib.Path(path)
    file = path / "config.json" if path.is_dir() else path
    if not file.exists():
        raise ConfigError(f"{file} does not exist")
    raw = json.loads(file.read_text())
    cfg = dict(raw.get("text_config", raw))
    names = raw.get("architectures") or cfg.get("architectures")
    if not names:
        raise ConfigError(f"{file} names no architectures")
    arch = resolve(names)
    cfg["architectures"] = [arch.name]
    return arch, arch.read_config(cfg), cfg
