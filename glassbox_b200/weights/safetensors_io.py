"""A small reader and writer for the safetensors container.

File = 8-byte little-endian header length, a JSON header {name: {dtype, shape, data_offsets}},
then the raw little-endian tensor bytes. The reader memory-maps the file and hands out
torch views without copying; every offset is checked against the file size first.
Glassbox maps ``model.safetensors`` the same way (crates/glassbox-core/src/load.rs:88-96)
and accepts F32, F16 and BF16 (load.rs:12-28); integer tables are accepted here as well.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import numpy as np
import torch


class WeightsError(ValueError):
    """A weights file that cannot be used; the message lists everything wrong with it."""


_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8), "F64": (torch.float64, 8),
    "U8": (torch.uint8, 1), "I8": (torch.int8, 1), "I16": (torch.int16, 2), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """Read-only view of one safetensors file. Tensors are views into the mapping and stay
    valid while this object is alive."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except FileNotFoundError:
            raise WeightsError(f"{path}: no such file") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8 or hlen > (1 << 30):
            raise WeightsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise WeightsError(f"{path}: header must be a JSON object")
        self._base = 8 + hlen
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        self._buf = np.frombuffer(self._map, dtype=np.uint8)
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        data_size = size - self._base
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (lo, hi) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise WeightsError(f"{path}: malformed header entry for {name!r}") from None
            if dtype not in _DTYPES:
                raise WeightsError(f"{path}: tensor {name!r} has unsupported dtype {dtype}")
            want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dtype][1] if shape else _DTYPES[dtype][1]
            if not (0 <= lo <= hi <= data_size) or hi - lo != want:
                raise WeightsError(f"{path}: tensor {name!r} {dtype}{list(shape)} has data offsets [{lo}, {hi}) "
                                   f"which do not match its size or the file ({data_size} data bytes)")
            self.entries[name] = (dtype, shape, lo, hi)

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, lo, hi = self.entries[name]
        raw = self._buf[self._base + lo:self._base + hi]
        tdtype = _DTYPES[dtype][0]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; callers copy before writing
            t = torch.from_numpy(raw)
        return t.view(tdtype).reshape(shape)

    def close(self) -> None:
        self._buf = None
        try:
            if self._map is not None:
                self._map.close()
        except BufferError:
            pass  # a view is still alive somewhere; the mapping goes when it does
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write ``tensors`` (CPU, contiguous) in name order; data is 8-byte aligned."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightsError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)
