"""Random weights from a configuration and a seed; can write a whole model folder
(config.json + model.safetensors) so that the loader path runs on the same numbers.

Distributions: matrices N(0, std), norm weights 1, conv taps N(0, conv_std), expert bias
N(0, bias_std).  Tensors are drawn in float32 in declaration order from one seeded CPU generator,
then stored as ``dtype`` (expert bias always float32, as checkpoints store it)."""
from __future__ import annotations

import json
import pathlib

import torch

from ..parts.spec import INIT_BIAS, INIT_CONV, INIT_NORMAL, INIT_ONES, KEEP_F32, KEEP_I32

DEFAULT_STD, DEFAULT_CONV_STD, DEFAULT_BIAS_STD = 0.02, 0.1, 0.01


def random_tensors(model, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = DEFAULT_STD,
                   conv_std: float = DEFAULT_CONV_STD, bias_std: float = DEFAULT_BIAS_STD,
                   device="cpu", fan_in_scaled: bool = False, norm_jitter: float = 0.0):
    """name -> tensor (stored shape) for everything ``model`` declares.

    ``fan_in_scaled`` draws matrices with std 1/sqrt(fan_in), so that every layer moves the
    residual stream by about its own size (tests use it: with std 0.02 the layers barely change
    the embedding).  ``norm_jitter`` draws norm weights as 1 + N(0, jitter) instead of exactly 1."""
    gen = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for _, spec in model.declare(lambda name: False):
        shape = spec.stored_shape
        if spec.keep == KEEP_I32:
            t = torch.zeros(shape, dtype=torch.int32, device=device)
        elif spec.init == INIT_ONES:
            t = torch.ones(shape, dtype=torch.float32, device=device)
            if norm_jitter:
                t = t + torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * norm_jitter
        else:
            s = {INIT_NORMAL: std, INIT_CONV: conv_std, INIT_BIAS: bias_std}[spec.init]
            if fan_in_scaled and spec.init == INIT_NORMAL and len(shape) >= 2:
                s = shape[-1] ** -0.5
            t = torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * s
        if spec.keep not in (KEEP_F32, KEEP_I32):
            t = t.to(dtype)
        out[spec.name] = t
    return out


def write_model_folder(folder, config_json: dict, tensors: dict) -> pathlib.Path:
    from .safetensors_io import write_safetensors
    folder = pathlib.Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config_json, indent=1))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder
