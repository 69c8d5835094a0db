"""Reading and writing safetensors files.

Format, as the reference reads it (crates/janus-engine/src/formats/safetensors.rs:36-120):
8 bytes little-endian header length, a JSON header `{name: {dtype, shape,
data_offsets}}` (the `__metadata__` entry is skipped), then the raw tensor
bytes; offsets are relative to the end of the header and are bounds-checked.
The file is memory-mapped; tensors are views into the mapping.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from typing import Dict, List, Tuple

import torch


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors file."""


_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_DTYPE_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One memory-mapped file; `tensor(name)` returns a CPU view (zero-copy)."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._file = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open '{path}': {e}") from e
        size = self._file.seek(0, 2)
        if size < 8:
            raise SafetensorsError(f"'{path}': file too small for a safetensors header ({size} bytes)")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if 8 + header_len > size:
            raise SafetensorsError(
                f"'{path}': header length {header_len} exceeds the file size {size} (truncated file?)")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"'{path}': header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"'{path}': header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + header_len
        data_size = size - self._data_start
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                dtype_name, shape, (begin, end) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(f"'{path}': malformed header entry for '{name}'") from e
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"'{path}': tensor '{name}' has unsupported dtype {dtype_name}")
            dtype, width = _DTYPES[dtype_name]
            count = 1
            for s in shape:
                count *= int(s)
            if begin < 0 or end < begin or end > data_size:
                raise SafetensorsError(
                    f"'{path}': tensor '{name}' data [{begin}, {end}) lies outside the file's "
                    f"{data_size} data bytes (truncated file?)")
            if end - begin != count * width:
                raise SafetensorsError(
                    f"'{path}': tensor '{name}' of shape {list(shape)} and dtype {dtype_name} needs "
                    f"{count * width} bytes but its offsets give {end - begin}")
            self._entries[name] = (dtype, shape, begin, end)

    def names(self) -> List[str]:
        return list(self._entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self._entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        buf = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the mapping is read-only; tensors are not written to
            return torch.frombuffer(buf, dtype=dtype).view(shape)


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] = None) -> None:
    """Write `tensors` (CPU, contiguous) in name order, data aligned to 8 bytes."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _DTYPE_NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _DTYPE_NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy())
