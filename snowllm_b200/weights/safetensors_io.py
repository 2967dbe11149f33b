"""Reading and writing safetensors files: 8-byte little-endian header length, a JSON header
(name -> dtype, shape, data_offsets), then the raw bytes (snowllm/checkpoint/reader.py:42-76).
A folder may hold one ``model.safetensors``, or shards named by ``model.safetensors.index.json``
(snowllm/checkpoint/reader.py:223-230)."""
from __future__ import annotations

import json
import mmap
import warnings
import pathlib
import struct

import torch

from ..errors import WeightError

DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
          "I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8,
          "U8": torch.uint8, "BOOL": torch.bool}
NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path):
        self.path = pathlib.Path(path)
        with open(self.path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise WeightError(f"{self.path}: not a safetensors file (too short)")
            (n,) = struct.unpack("<Q", head)
            try:
                self.header = json.loads(f.read(n))
            except (ValueError, UnicodeDecodeError) as e:
                raise WeightError(f"{self.path}: unreadable safetensors header: {e}") from e
            self.base = 8 + n
            self.header.pop("__metadata__", None)
            self._file = open(self.path, "rb")
            size = self.path.stat().st_size
            self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self):
        return list(self.header)

    def meta(self, name):
        m = self.header[name]
        if m["dtype"] not in DTYPES:
            raise WeightError(f"{self.path}: tensor {name} has unsupported dtype {m['dtype']}")
        return DTYPES[m["dtype"]], tuple(m["shape"])

    def tensor(self, name) -> torch.Tensor:
        """A CPU tensor that views the mapped file (copy it before the file is closed)."""
        dtype, shape = self.meta(name)
        lo, hi = self.header[name]["data_offsets"]
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        if hi - lo != count * torch.empty((), dtype=dtype).element_size():
            raise WeightError(f"{self.path}: tensor {name} holds {hi - lo} bytes, shape {shape} "
                              f"of {dtype} needs {count * torch.empty((), dtype=dtype).element_size()}")
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)    # the map is read-only; nobody writes to it
            return torch.frombuffer(self._map, dtype=dtype, count=count,
                                    offset=self.base + lo).reshape(shape)

    def close(self):
        # tensors handed out may still view the map; dropping our references is enough
        self._map = None
        self._file.close()


class Checkpoint:
    """All tensors of a model folder by name."""

    def __init__(self, folder):
        folder = pathlib.Path(folder)
        index = folder / "model.safetensors.index.json"
        self.files: dict[str, SafetensorsFile] = {}
        self.where: dict[str, str] = {}
        if index.exists():
            for name, shard in json.loads(index.read_text())["weight_map"].items():
                if shard not in self.files:
                    self.files[shard] = SafetensorsFile(folder / shard)
                self.where[name] = shard
        else:
            single = folder / "model.safetensors"
            if not single.exists():
                found = sorted(folder.glob("*.safetensors"))
                if not found:
                    raise WeightError(f"{folder} holds no .safetensors file")
                single = found[0]
            f = SafetensorsFile(single)
            self.files[single.name] = f
            self.where = {n: single.name for n in f.names()}

    def names(self):
        return list(self.where)

    def has(self, name) -> bool:
        return name in self.where

    def meta(self, name):
        return self.files[self.where[name]].meta(name)

    def read(self, name) -> torch.Tensor:
        if name not in self.where:
            raise WeightError(f"checkpoint has no tensor {name}")
        return self.files[self.where[name]].tensor(name)

    def close(self):
        for f in self.files.values():
            f.close()


def write_safetensors(path, tensors) -> None:
    """Write ``tensors`` (a dict, or an iterable of (name, tensor) that can be walked twice when
    given as a callable returning an iterator) in the order given."""
    items = tensors.items() if hasattr(tensors, "items") else tensors
    header, offset, order = {}, 0, []
    for name, t in items:
        if t.dtype not in NAMES:
            raise WeightError(f"cannot store dtype {t.dtype}")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
        order.append((name, t))
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-(8 + len(blob)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in order:
            if t.numel():
                f.write(t.detach().contiguous().cpu().reshape(-1).view(torch.uint8).numpy().tobytes())
