"""Reading and writing safetensors files, by tensor name.

The format: 8 bytes little-endian header length N, N bytes of JSON mapping each tensor
name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end
of the header), then the raw little-endian data.  The reader maps the file and hands out
tensors as views into the mapping (no copy until the caller moves them); a folder may hold
one ``model.safetensors`` or several shards named by ``model.safetensors.index.json``.
The reference reads GGUF the same way: name-keyed, shape-checked views into an mmap
(src/locus/model/gguf_load.hpp:34-48).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Callable, Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": torch.float32,
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F64": torch.float64,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def _itemsize(dt: torch.dtype) -> int:
    return torch.empty((), dtype=dt).element_size()


class SafetensorsFile:
    """One mapped safetensors file."""

    def __init__(self, path: str) -> None:
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._mm[:8])
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file")
        try:
            header = json.loads(self._mm[8 : 8 + n].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        self._data0 = 8 + n
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dt = _DTYPES[e["dtype"]]
                shape = tuple(int(s) for s in e["shape"])
                b, en = (int(v) for v in e["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: bad header entry for tensor {name}") from None
            numel = 1
            for s in shape:
                numel *= s
            if en - b != numel * _itemsize(dt) or b < 0 or self._data0 + en > size:
                raise SafetensorsError(f"{path}: tensor {name} has inconsistent offsets")
            self.entries[name] = (dt, shape, b, en)

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self.entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        buf = memoryview(self._mm)[self._data0 + b : self._data0 + e]
        with warnings.catch_warnings():
            # the mapping is read-only; the tensors are only ever copied from
            warnings.simplefilter("ignore", UserWarning)
            return torch.frombuffer(buf, dtype=dt).reshape(shape)

    def close(self) -> None:
        # views handed out keep the mapping alive; closing is best effort
        try:
            self._mm.close()
        except (BufferError, ValueError):
            pass
        self._f.close()


class ModelFiles:
    """All safetensors tensors of a model folder, by name."""

    def __init__(self, model_dir: str) -> None:
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f).get("weight_map", {})
            for name, fn in weight_map.items():
                self._where[name] = fn
            for fn in sorted(set(weight_map.values())):
                self._files[fn] = SafetensorsFile(os.path.join(model_dir, fn))
            for name, fn in self._where.items():
                if name not in self._files[fn].entries:
                    raise SafetensorsError(f"{index}: tensor {name} is not in {fn}")
        elif os.path.isfile(single):
            sf = SafetensorsFile(single)
            self._files["model.safetensors"] = sf
            for name in sf.names():
                self._where[name] = "model.safetensors"
        else:
            raise SafetensorsError(f"no model.safetensors (or index) in model folder: {model_dir}")

    def names(self) -> List[str]:
        return list(self._where)

    def info(self, name: str):
        return self._files[self._where[name]].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)

    def close(self) -> None:
        for f in self._files.values():
            f.close()


def write_safetensors(path: str, specs: Iterable[Tuple[str, Tuple[int, ...], torch.dtype]],
                      produce: Callable[[str], torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Write tensors one at a time: ``produce(name)`` is called in order, so a model larger
    than host memory can be written."""
    specs = list(specs)
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    for name, shape, dt in specs:
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * _itemsize(dt)
        header[name] = {"dtype": _NAMES[dt], "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape, dt in specs:
            t = produce(name)
            if tuple(t.shape) != tuple(shape) or t.dtype != dt:
                raise SafetensorsError(f"write: tensor {name} is {tuple(t.shape)} {t.dtype}, expected {shape} {dt}")
            t = t.detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
