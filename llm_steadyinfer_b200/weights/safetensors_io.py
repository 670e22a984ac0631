"""Reader and writer for the safetensors container: an 8-byte little-endian header
length, a JSON header {name: {dtype, shape, data_offsets}}, then raw little-endian
tensor bytes. The reference reads a custom .bin by pointer arithmetic into an mmap
(src/source/model/model.cpp:283-353, llama3.cpp:299-432); here tensors are found by
name and the file is mapped, not copied.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A mapped safetensors file. ``tensor(name)`` returns a CPU view of the mapping."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        self._base = 8 + n
        for name, e in header.items():
            dt = e.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            shape = tuple(int(s) for s in e["shape"])
            b, en = (int(x) for x in e["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty(0, dtype=_DTYPES[dt]).element_size()
            if en - b != want or self._base + en > size or b < 0:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} spans bytes [{b},{en}) but its shape {shape} "
                    f"and dtype {dt} need {want} bytes (file has {size - self._base} data bytes)")
            self._entries[name] = (_DTYPES[dt], shape, b, en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> Iterable[str]:
        return self._entries.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b, e = self._entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        buf = memoryview(self._mm)[self._base + b: self._base + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # the mapping is read-only; tensors are only read
            t = torch.frombuffer(buf, dtype=dt)
        return t.view(shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
