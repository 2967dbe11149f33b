"""From a model folder to a model ready to step (the role of snowllm/checkpoint/loader.py:186-261)."""
from __future__ import annotations

import pathlib

import torch

from .config.registry import read_config_json
from .errors import ConfigError
from .model import Model
from .weights.loader import load_folder, load_tensors
from .weights.random_init import random_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ConfigError(f"dtype {dtype!r}: want bfloat16 or float32") from None


def build_model(path_or_config, dtype="bfloat16") -> Model:
    """An unbound model (parts built, no weights) from a folder, a config.json or a raw dict."""
    dtype = parse_dtype(dtype)
    if isinstance(path_or_config, dict):
        from .config.registry import resolve
        raw = dict(path_or_config.get("text_config", path_or_config))
        arch = resolve(path_or_config.get("architectures") or raw.get("architectures"))
        raw["architectures"] = [arch.name]
        config = arch.read_config(raw)
    else:
        arch, config, _ = read_config_json(path_or_config)
    return Model(arch.model_spec(config), dtype, config=config)


def load(path, dtype="bfloat16", device="cuda") -> Model:
    """Model of the folder ``path`` (config.json + safetensors) with its weights on ``device``."""
    model = build_model(path, dtype)
    load_folder(model, pathlib.Path(path), device)
    return model


def load_random(config, seed: int = 0, dtype="bfloat16", device="cuda", **init) -> Model:
    """Model with seeded random weights drawn straight on ``device`` (no file)."""
    model = build_model(config, dtype)
    tensors = random_tensors(model, seed, parse_dtype(dtype), device=device, **init)
    load_tensors(model, tensors, device)
    return model
