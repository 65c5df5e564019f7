"""Weights from safetensors by tensor name.

The reference walks the GGUF tensor table, maps names to slots and converts dtypes
as it goes (internal/engine/engine.go:736-1104), and notices a missing tensor only
when inference starts (engine.go:1316-1324).  Here the model says which names and
shapes it needs, and one error lists everything that is wrong with the file.

Kept as stored where possible: bfloat16 stays bfloat16, a tensor stored in 32-bit
stays in 32-bit, float16 becomes bfloat16, integer tables become int32.  The reference
converts every tensor to the precision of its path as it loads
(internal/engine/engine.go:787-802); `convert_to` asks for the same: floating-point
tensors are rounded to that dtype at load, except those a part wants in full precision
(norm gains, which the reference promotes to 32-bit, engine.go:788-792).  Tensors that
the model does not name are an error by default, as missing ones are; `unexpected="warn"`
lists them in a warning instead (the reference skips what it does not know,
engine.go:867-870).
"""
from __future__ import annotations

import json
import warnings
from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile
from .spec import WeightSpec


class WeightsError(ValueError):
    """The checkpoint does not hold what the model needs; lists every fault."""

    def __init__(self, where, missing, unexpected, wrong_shape, other=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.other = list(other)
        lines = [f"{where}: the checkpoint does not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " +
                         "; ".join(f"{n}: expected {list(e)}, found {list(f)}" for n, e, f in self.wrong_shape))
        for msg in self.other:
            lines.append("  " + msg)
        super().__init__("\n".join(lines))


def _open_files(folder: Path) -> list[SafetensorsFile]:
    single = folder / "model.safetensors"
    index = folder / "model.safetensors.index.json"
    if single.is_file():
        return [SafetensorsFile(single)]
    if index.is_file():
        shards = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        return [SafetensorsFile(folder / s) for s in shards]
    raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")


def _keep_dtype(t: torch.Tensor, spec: WeightSpec, convert_to: torch.dtype | None = None) -> torch.Tensor:
    if spec.integer:
        return t.to(torch.int32)
    if convert_to is not None and t.dtype.is_floating_point and not spec.full_precision:
        if convert_to == torch.float32 and t.dtype == torch.bfloat16:
            return t                  # every bfloat16 value is a float32 value: the 32-bit kernels read it as it is
        return t.to(convert_to)
    if t.dtype in (torch.float32, torch.bfloat16):
        return t
    if t.dtype in (torch.float16,):
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    raise SafetensorsError(f"dtype {t.dtype} is not a weight dtype")


class _Uploader:
    """Host memory that is mapped from a file goes to the device through two pinned buffers in turn: while one
    buffer's copy to the device runs (asynchronously, on a stream of its own), the next piece of the file is read
    into the other.  The reference maps its file and hands each tensor to the device as it walks the table
    (internal/gguf/reader.go:16-35, internal/engine/engine.go:736-806)."""

    CHUNK = 64 << 20

    def __init__(self, device):
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device)
        self.buffers = [torch.empty(self.CHUNK, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.free = [torch.cuda.Event(), torch.cuda.Event()]
        self.turn = 0

    def upload(self, src: torch.Tensor) -> torch.Tensor:
        src = src.contiguous()
        dst = torch.empty(src.shape, dtype=src.dtype, device=self.device)
        if src.numel() == 0:
            return dst
        src_bytes, dst_bytes = src.reshape(-1).view(torch.uint8), dst.reshape(-1).view(torch.uint8)
        for lo in range(0, src_bytes.numel(), self.CHUNK):
            n = min(self.CHUNK, src_bytes.numel() - lo)
            buf = self.buffers[self.turn]
            self.free[self.turn].synchronize()                  # the copy that last used this buffer has left it
            buf[:n].copy_(src_bytes[lo:lo + n])
            with torch.cuda.stream(self.stream):
                dst_bytes[lo:lo + n].copy_(buf[:n], non_blocking=True)
                self.free[self.turn].record(self.stream)
            self.turn ^= 1
        return dst

    def finish(self) -> None:
        self.stream.synchronize()
        torch.cuda.current_stream(self.device).wait_stream(self.stream)


def load_weights(folder, table: dict[str, WeightSpec], device, convert_to: torch.dtype | None = None,
                 unexpected: str = "error") -> dict[str, torch.Tensor]:
    """Every tensor of `table` on `device`.  A name with a `fallback` that is absent
    from the file is left out of the result (the part then reads the fallback).
    convert_to: round floating-point tensors to this dtype at load (None: keep them as stored).
    unexpected: "error" (tensors the model does not name are a fault like the others), "warn" or "ignore"."""
    if unexpected not in ("error", "warn", "ignore"):
        raise ValueError(f"unexpected must be 'error', 'warn' or 'ignore', found {unexpected!r}")
    folder = Path(folder)
    files = _open_files(folder)
    where: dict[str, SafetensorsFile] = {}
    other = []
    for f in files:
        for name in f.names():
            if name in where:
                other.append(f"tensor {name} appears in both {where[name].path.name} and {f.path.name}")
            where[name] = f
    missing, wrong = [], []
    for name, spec in table.items():
        if name not in where:
            if spec.fallback is not None and spec.fallback in table:
                continue
            missing.append(name)
        elif where[name].shape(name) != tuple(spec.shape):
            wrong.append((name, tuple(spec.shape), where[name].shape(name)))
        elif spec.integer == where[name].dtype(name).is_floating_point:
            other.append(f"tensor {name} has dtype {where[name].dtype(name)}, expected "
                         f"{'an integer' if spec.integer else 'a floating-point'} type")
    extra = [n for n in where if n not in table]
    if missing or wrong or other or (extra and unexpected == "error"):
        raise WeightsError(folder, missing, extra, wrong, other)
    if extra and unexpected == "warn":
        warnings.warn(f"{folder}: {len(extra)} tensors that the model does not name are skipped: " + ", ".join(sorted(extra)))
    out = {}
    uploader = _Uploader(device) if torch.device(device).type == "cuda" else None
    for name, spec in table.items():
        if name in where:
            stored = where[name].tensor(name)
            if uploader is None:
                out[name] = _keep_dtype(stored, spec, convert_to).to(device).contiguous()
            else:
                out[name] = uploader.upload(stored)       # as stored; converted on the device below
    if uploader is not None:
        uploader.finish()
        for name in list(out):
            out[name] = _keep_dtype(out[name], table[name], convert_to).contiguous()
    for f in files:
        f.close()
    return out
