"""Reading and writing the safetensors container.

Layout of a file: an unsigned 64-bit little-endian header length, a JSON header that
maps each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header), then the raw little-endian data.  A model folder
has either one ``model.safetensors`` or several shards listed by
``model.safetensors.index.json`` (``weight_map``: tensor name -> shard file).
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable

import torch


class WeightsError(RuntimeError):
    """A weights file or folder that cannot be used, with the reason."""


_TORCH_DTYPE = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_ST_NAME = {v: k for k, v in _TORCH_DTYPE.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str            # safetensors dtype string
    shape: tuple
    begin: int            # absolute byte offsets in the file
    end: int
    file: Path


class SafetensorsFile:
    """One memory-mapped safetensors file; tensors come out as CPU views of the map."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except OSError as e:
            raise WeightsError(f"{self.path}: cannot open ({e.strerror})") from None
        size = self.path.stat().st_size
        if size < 8:
            raise WeightsError(f"{self.path}: too short to be a safetensors file ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise WeightsError(f"{self.path}: header length {hlen} does not fit the file "
                               f"({size} bytes)")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightsError(f"{self.path}: header is not valid JSON ({e})") from None
        base = 8 + hlen
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape = info["dtype"], tuple(int(s) for s in info["shape"])
                a, b = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise WeightsError(f"{self.path}: malformed header entry for {name!r}") from None
            if dtype not in _TORCH_DTYPE:
                raise WeightsError(f"{self.path}: tensor {name!r} has unsupported dtype {dtype}")
            n = 1
            for s in shape:
                n *= s
            want = n * torch.empty((), dtype=_TORCH_DTYPE[dtype]).element_size()
            if a < 0 or b < a or base + b > size or b - a != want:
                raise WeightsError(
                    f"{self.path}: tensor {name!r} ({dtype}{list(shape)}) has data range "
                    f"[{a},{b}) but needs {want} bytes within a file of {size} bytes (truncated?)")
            self.entries[name] = TensorEntry(name, dtype, shape, base + a, base + b, self.path)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        n = 1
        for s in e.shape:
            n *= s
        if n == 0:
            return torch.empty(e.shape, dtype=_TORCH_DTYPE[e.dtype])
        t = torch.frombuffer(self._map, dtype=_TORCH_DTYPE[e.dtype], count=n, offset=e.begin)
        return t.reshape(e.shape)

    def close(self) -> None:
        # views handed out keep the map alive through the buffer protocol; closing
        # is attempted and ignored when views still exist
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass
        self._fh.close()


def open_model_files(folder) -> list[SafetensorsFile]:
    """The safetensors files of a model folder (one file, or the shards of the index)."""
    folder = Path(folder)
    index = folder / "model.safetensors.index.json"
    single = folder / "model.safetensors"
    if index.is_file():
        try:
            wm = json.loads(index.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError) as e:
            raise WeightsError(f"{index}: cannot read weight_map ({e})") from None
        return [SafetensorsFile(folder / f) for f in sorted(set(wm.values()))]
    if single.is_file():
        return [SafetensorsFile(single)]
    raise WeightsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")


def write_safetensors(path, tensors: Iterable[tuple[str, tuple, torch.dtype, object]]) -> None:
    """Writes tensors given as (name, shape, dtype, producer); ``producer()`` returns the
    CPU tensor when its turn comes, so that only one tensor is held at a time."""
    items = list(tensors)
    header, off = {}, 0
    for name, shape, dtype, _ in items:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        header[name] = {"dtype": _ST_NAME[dtype], "shape": [int(s) for s in shape],
                        "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape, dtype, producer in items:
            t = producer().contiguous()
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise WeightsError(f"write_safetensors: producer of {name!r} returned "
                                   f"{t.dtype}{list(t.shape)}, expected {dtype}{list(shape)}")
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
