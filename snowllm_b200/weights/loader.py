"""Weights by tensor name: what the model declares against what the folder holds.

Every mismatch (missing tensors, tensors nothing asked for, wrong shapes, unusable dtypes) is
gathered into one WeightError.  Tensors go to the device in the dtype their spec asks for:
matrices in the compute dtype, small vectors that the file stores as float32 stay float32,
integer tables as int32 (snowllm/models/lfm2/weights.py:58-96; errors
snowllm/checkpoint/reader.py:57-61, 247-248)."""
from __future__ import annotations

import torch

from ..errors import WeightError
from ..parts.spec import KEEP_COMPUTE, KEEP_F32, KEEP_I32, KEEP_SMALL, TensorSpec
from .safetensors_io import Checkpoint

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)


def kept_dtype(spec: TensorSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.keep == KEEP_I32:
        return torch.int32
    if spec.keep == KEEP_F32:
        return torch.float32
    if spec.keep == KEEP_SMALL and stored in (torch.float32, torch.float64):
        return torch.float32
    return compute


def check_against(declared: list[TensorSpec], names, meta) -> None:
    """Raise one WeightError that lists everything wrong, or return."""
    wanted = {s.name: s for s in declared}
    have = set(names)
    missing = sorted(n for n in wanted if n not in have)
    unexpected = sorted(n for n in have if n not in wanted)
    wrong = []
    for n, s in wanted.items():
        if n not in have:
            continue
        dtype, shape = meta(n)
        if tuple(shape) not in (tuple(s.stored_shape), tuple(s.shape)):
            wrong.append(f"{n}: shape {tuple(shape)}, want {tuple(s.stored_shape)}")
        elif s.keep == KEEP_I32 and dtype in _FLOATS:
            wrong.append(f"{n}: dtype {dtype}, want an integer table")
        elif s.keep != KEEP_I32 and dtype not in _FLOATS:
            wrong.append(f"{n}: dtype {dtype}, want a float tensor")
    if missing or unexpected or wrong:
        def some(xs):
            return ", ".join(xs[:12]) + (f", ... ({len(xs)} in all)" if len(xs) > 12 else "")
        parts = []
        if missing:
            parts.append(f"missing tensors: {some(missing)}")
        if unexpected:
            parts.append(f"unexpected tensors: {some(unexpected)}")
        if wrong:
            parts.append(f"wrong shapes or dtypes: {some(wrong)}")
        raise WeightError("checkpoint does not match the model: " + "; ".join(parts))


def load_into(model, read, names, meta, has, device) -> None:
    """Declare, check, then bind part by part.  ``read(name)`` gives a CPU (or device) tensor."""
    declared = model.declare(has)
    check_against([s for _, s in declared], names, meta)
    by_part: dict[int, tuple[object, dict]] = {}
    for part, spec in declared:
        t = read(spec.name)
        dtype = kept_dtype(spec, t.dtype, model.dtype)
        t = t.to(device=device, dtype=dtype).reshape(spec.shape)
        by_part.setdefault(id(part), (part, {}))[1][spec.local] = t
    for part, tensors in by_part.values():
        part.bind(tensors)
    model.bound_bytes = {key: {local: t.numel() * t.element_size() for local, t in tensors.items()}
                         for key, (_, tensors) in by_part.items()}
    model.finish_binding()


def load_folder(model, folder, device) -> None:
    ck = Checkpoint(folder)
    try:
        load_into(model, ck.read, ck.names(), ck.meta, ck.has, device)
    finally:
        ck.close()


def load_tensors(model, tensors: dict, device) -> None:
    """Bind from an in-memory dict of name -> tensor (the random-weights mode without a file)."""
    load_into(model, tensors.__getitem__, list(tensors),
              lambda n: (tensors[n].dtype, tuple(tensors[n].shape)), tensors.__contains__, device)
