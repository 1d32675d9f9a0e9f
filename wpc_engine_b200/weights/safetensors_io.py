"""Reading and writing the safetensors container: 8 bytes of little-endian header length, a
JSON header (`name -> {dtype, shape, data_offsets}`), then the tensors' bytes.

The reference reads the same container through a crate (wpc-runtime/src/weights.rs:125-177)
and, for sharded checkpoints, `model.safetensors.index.json` (weights.rs:189-264).  Here a
file is memory-mapped and a tensor becomes a torch view of its bytes, so a 16-bit tensor stays
16-bit and a 32-bit one stays 32-bit until the loader decides otherwise.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8), "F64": (torch.float64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class WeightFileError(RuntimeError):
    """A weight file that cannot be read."""


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightFileError(f"cannot open {path}: {e}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightFileError(f"{path}: too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise WeightFileError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFileError(f"{path}: malformed header: {e}") from None
        header.pop("__metadata__", None)
        self._data_start = 8 + hlen
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, meta in header.items():
            dtype, shape = meta["dtype"], tuple(int(s) for s in meta["shape"])
            lo, hi = meta["data_offsets"]
            if dtype in _DTYPES:
                want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dtype][1]
                if hi - lo != want or self._data_start + hi > size:
                    raise WeightFileError(f"{path}: tensor {name} has {hi - lo} bytes, its shape needs {want}")
            self.entries[name] = (dtype, shape, lo, hi)

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype_name(self, name: str) -> str:
        return self.entries[name][0]

    def read(self, name: str) -> torch.Tensor:
        """The tensor in its stored type, as a host tensor that owns a copy of the bytes."""
        dtype, shape, lo, hi = self.entries[name]
        if dtype not in _DTYPES:
            raise WeightFileError(f"{self.path}: tensor {name} has unsupported dtype {dtype}")
        tdtype, _ = _DTYPES[dtype]
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=hi - lo, offset=self._data_start + lo)
        return torch.from_numpy(buf.copy()).view(tdtype).reshape(shape)

    def close(self):
        try:
            self._mm.close()
        finally:
            self._f.close()


class ModelFiles:
    """`model.safetensors`, or the shards that `model.safetensors.index.json` lists."""

    def __init__(self, folder: str):
        single = os.path.join(folder, "model.safetensors")
        index = os.path.join(folder, "model.safetensors.index.json")
        self.files: Dict[str, SafetensorsFile] = {}
        self.where: Dict[str, str] = {}
        if os.path.exists(single):
            f = SafetensorsFile(single)
            self.files[single] = f
            self.where = {n: single for n in f.names()}
        elif os.path.exists(index):
            try:
                with open(index) as fh:
                    weight_map = json.load(fh)["weight_map"]
            except (KeyError, json.JSONDecodeError) as e:
                raise WeightFileError(f"{index}: no usable weight_map: {e}") from None
            for name, shard in weight_map.items():
                path = os.path.join(folder, shard)
                if path not in self.files:
                    self.files[path] = SafetensorsFile(path)
                if name not in self.files[path].entries:
                    raise WeightFileError(f"{index} places {name} in {shard}, which does not hold it")
                self.where[name] = path
        else:
            raise WeightFileError(f"{folder} holds neither model.safetensors nor model.safetensors.index.json")

    def names(self) -> List[str]:
        return list(self.where)

    def shape(self, name: str):
        return self.files[self.where[name]].shape(name)

    def dtype_name(self, name: str) -> str:
        return self.files[self.where[name]].dtype_name(name)

    def read(self, name: str) -> torch.Tensor:
        return self.files[self.where[name]].read(name)

    def close(self):
        for f in self.files.values():
            f.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Writes host tensors in the order given."""
    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    header = {}
    off = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise WeightFileError(f"cannot store dtype {t.dtype} of {name}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
