"""Reader and writer of the safetensors container: an 8-byte little-endian header length,
a JSON header ``{name: {dtype, shape, data_offsets}}`` and the raw little-endian data.

The reference reads GGUF through a memory map and looks tensors up by name in a map
merged over the parts of a split file (src/models/qwen2/loader.rs:224-251); this file
plays that role for the safetensors container, including a sharded checkpoint's
``model.safetensors.index.json``.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Iterable, Mapping

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    dtype_name: str
    shape: tuple[int, ...]
    begin: int
    end: int
    file: str


class SafetensorsFile:
    """One file, memory-mapped; tensors are views into the map until they are copied."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header")
        self._file = open(path, "rb")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        if header_len > size - 8:
            raise SafetensorsError(
                f"{path}: header length {header_len} exceeds the file size {size} (truncated file?)")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: the header is not valid JSON ({e})") from None
        self._data_start = 8 + header_len
        data_size = size - self._data_start
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype_name = info["dtype"]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for '{name}'") from None
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype_name}")
            dtype = _DTYPES[dtype_name]
            count = 1
            for s in shape:
                count *= s
            want = count * torch.empty((), dtype=dtype).element_size()
            if begin < 0 or end < begin or end > data_size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' lies at bytes [{begin}, {end}) but the data section "
                    f"has {data_size} bytes (truncated file?)")
            if end - begin != want:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' of shape {list(shape)} {dtype_name} needs {want} "
                    f"bytes, the header gives {end - begin}")
            self.entries[name] = TensorEntry(name, dtype, dtype_name, shape, begin, end, path)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> list[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns its memory (copied out of the map)."""
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        view = memoryview(self._map)[self._data_start + e.begin:self._data_start + e.end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # the map is read-only; the clone below owns its data
            flat = torch.frombuffer(view, dtype=e.dtype)
        return flat.reshape(e.shape).clone()

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass            # a view is still alive; the map goes with it
            self._map = None
        self._file.close()


class Checkpoint:
    """All tensors of a model folder, whether in ``model.safetensors`` or in shards."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        files: list[str]
        if os.path.exists(single):
            files = [single]
        elif os.path.exists(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f).get("weight_map", {})
            files = sorted({os.path.join(folder, v) for v in weight_map.values()})
            if not files:
                raise SafetensorsError(f"{index}: 'weight_map' is empty")
        else:
            raise SafetensorsError(
                f"{folder}: neither model.safetensors nor model.safetensors.index.json found")
        self.files = [SafetensorsFile(p) for p in files]
        self.where: dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name in f.entries:
                if name in self.where:
                    raise SafetensorsError(
                        f"tensor '{name}' appears in both {self.where[name].path} and {f.path}")
                self.where[name] = f

    def names(self) -> list[str]:
        return list(self.where)

    def entry(self, name: str) -> TensorEntry:
        return self.where[name].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def save_file(tensors: Mapping[str, torch.Tensor], path: str,
              metadata: Mapping[str, str] | None = None) -> None:
    """Writes ``tensors`` (CPU, any listed dtype) in name order."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which safetensors lacks")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(_raw_bytes(t))
    os.replace(tmp, path)


def _raw_bytes(t: torch.Tensor) -> bytes:
    if t.numel() == 0:
        return b""
    return t.reshape(-1).view(torch.uint8).numpy().tobytes()


def load_all(folder: str, names: Iterable[str] | None = None) -> dict[str, torch.Tensor]:
    ck = Checkpoint(folder)
    try:
        wanted = list(names) if names is not None else ck.names()
        return {n: ck.tensor(n) for n in wanted}
    finally:
        ck.close()
