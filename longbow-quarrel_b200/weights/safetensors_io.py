"""Reading and writing the safetensors container: an 8-byte little-endian header
length, a JSON header {name: {dtype, shape, data_offsets}}, then raw little-endian
tensor bytes.  It takes the place of the reference's GGUF reader
(internal/gguf/reader.go:16-336), which also maps the file and hands out tensors
by name.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
          "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
          "U8": torch.uint8, "BOOL": torch.bool}
NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A mapped safetensors file; `tensor(name)` is a CPU view of the mapping."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise SafetensorsError(f"{self.path}: no such file")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: truncated (only {size} bytes)")
        self._fh = open(self.path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)
        (n,) = struct.unpack("<Q", self._map[:8])
        if 8 + n > size:
            raise SafetensorsError(f"{self.path}: header of {n} bytes does not fit in a file of {size} bytes")
        try:
            header = json.loads(self._map[8:8 + n].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{self.path}: header is not valid JSON: {exc}") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + n
        self.entries: dict[str, dict] = {}
        for name, info in header.items():
            dtype = info.get("dtype")
            if dtype not in DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unknown dtype {dtype!r}")
            lo, hi = info["data_offsets"]
            numel = 1
            for s in info["shape"]:
                numel *= int(s)
            want = numel * torch.empty((), dtype=DTYPES[dtype]).element_size()
            if hi - lo != want:
                raise SafetensorsError(f"{self.path}: tensor {name!r} of shape {info['shape']} {dtype} needs "
                                       f"{want} bytes, offsets give {hi - lo}")
            if lo < 0 or self._base + hi > size:
                raise SafetensorsError(f"{self.path}: tensor {name!r} data [{lo}, {hi}) lies outside the file "
                                       f"(truncated?)")
            self.entries[name] = info

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(int(s) for s in self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return DTYPES[self.entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        info = self.entries[name]
        lo, hi = info["data_offsets"]
        dtype = DTYPES[info["dtype"]]
        shape = self.shape(name)
        if hi == lo:
            return torch.empty(shape, dtype=dtype)
        count = (hi - lo) // torch.empty((), dtype=dtype).element_size()
        return torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._base + lo).reshape(shape)

    def close(self) -> None:
        # Tensors handed out keep the mapping alive; closing only drops our handle.
        self._fh.close()


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    header, offset, blobs = {}, 0, []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(head)))
        fh.write(head)
        for raw in blobs:
            fh.write(raw)
