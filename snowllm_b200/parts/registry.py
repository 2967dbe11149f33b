"""Registries of part kinds: mixers, feed-forwards, norms, position encodings, block
arrangements, embeddings and output heads.

A ``ModelSpec`` names parts by kind; the model builder looks each kind up here.  Registering a
new kind (``register_mixer("my_mixer", MyMixer)``) is all it takes for a new architecture's
``ModelSpec`` to use it; no file of the framework changes.
"""
from __future__ import annotations

from ..errors import ConfigError

_REGISTRIES: dict[str, dict[str, type]] = {
    "mixer": {}, "ffn": {}, "norm": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


def _register(family: str, kind: str, cls: type) -> type:
    _REGISTRIES[family][kind] = cls
    return cls


def register_mixer(kind, cls): return _register("mixer", kind, cls)
def register_ffn(kind, cls): return _register("ffn", kind, cls)
def register_norm(kind, cls): return _register("norm", kind, cls)
def register_position(kind, cls): return _register("position", kind, cls)
def register_block(kind, cls): return _register("block", kind, cls)
def register_embedding(kind, cls): return _register("embedding", kind, cls)
def register_head(kind, cls): return _register("head", kind, cls)


def lookup(family: str, kind: str) -> type:
    _load_builtin()
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "none"
        raise ConfigError(f"no {family} of kind {kind!r} is registered (known: {known})") from None


def kinds(family: str) -> list[str]:
    _load_builtin()
    return sorted(_REGISTRIES[family])


def _load_builtin() -> None:
    from . import attention, block, embedding, ffn_dense, ffn_moe, norm, position, short_conv  # noqa: F401
