"""Reading and writing safetensors files, without any helper library.

File format: 8 bytes little-endian header length N, N bytes of JSON mapping a tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the byte after the
header), then the payload.

Reference parity: ``src/core/safetensor.cpp:447-552`` (open, header length, JSON object) and
``safetensor.cpp:283-378,527-549`` (per-entry checks: known dtype, offsets ordered and inside the
payload, byte size equal to numel times item size, at least one element, no two tensors overlap).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import numpy as np
import torch


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors file."""


# name -> (item size, torch dtype, numpy carrier dtype)
_DTYPES = {
    "F64": (8, torch.float64, np.float64),
    "F32": (4, torch.float32, np.float32),
    "F16": (2, torch.float16, np.float16),
    "BF16": (2, torch.bfloat16, np.uint16),
    "I64": (8, torch.int64, np.int64),
    "I32": (4, torch.int32, np.int32),
    "I16": (2, torch.int16, np.int16),
    "I8": (1, torch.int8, np.int8),
    "U8": (1, torch.uint8, np.uint8),
    "BOOL": (1, torch.bool, np.bool_),
}
_TORCH_TO_NAME = {v[1]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: tuple
    begin: int
    end: int

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class SafetensorsFile:
    """A memory-mapped safetensors file.  ``tensor(name)`` returns a CPU tensor that views the map."""

    def __init__(self, path: str):
        self.path = os.fspath(path)
        size = os.path.getsize(self.path)
        if size < 8:
            raise SafetensorsError(f"'{self.path}': too small to hold a header length")
        self._fh = open(self.path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(f"'{self.path}': header length {header_len} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"'{self.path}': header is not valid JSON: {exc}") from exc
        if not isinstance(header, dict):
            raise SafetensorsError(f"'{self.path}': header must be a JSON object")
        self._payload = 8 + header_len
        payload_size = size - self._payload
        self.metadata = header.pop("__metadata__", None)
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            self.entries[name] = self._check_entry(name, info, payload_size)
        spans = sorted((e.begin, e.end, e.name) for e in self.entries.values())
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"'{self.path}': tensors '{n0}' and '{n1}' overlap")

    def _check_entry(self, name: str, info, payload_size: int) -> TensorEntry:
        where = f"'{self.path}': tensor '{name}'"
        if not isinstance(info, dict):
            raise SafetensorsError(f"{where}: entry must be an object")
        dtype = info.get("dtype")
        if dtype not in _DTYPES:
            raise SafetensorsError(f"{where}: unsupported dtype '{dtype}'")
        shape = info.get("shape")
        if not isinstance(shape, list) or not all(isinstance(s, int) and s >= 0 for s in shape):
            raise SafetensorsError(f"{where}: shape must be a list of non-negative integers")
        offsets = info.get("data_offsets")
        if (not isinstance(offsets, list) or len(offsets) != 2
                or not all(isinstance(o, int) and o >= 0 for o in offsets)):
            raise SafetensorsError(f"{where}: data_offsets must be two non-negative integers")
        begin, end = offsets
        if end < begin or end > payload_size:
            raise SafetensorsError(f"{where}: data_offsets [{begin}, {end}] fall outside the payload ({payload_size} bytes)")
        entry = TensorEntry(name, dtype, tuple(shape), begin, end)
        if entry.numel == 0:
            raise SafetensorsError(f"{where}: has no elements")
        if entry.numel * _DTYPES[dtype][0] != end - begin:
            raise SafetensorsError(
                f"{where}: {end - begin} bytes do not match shape {list(shape)} of {dtype}")
        return entry

    def names(self) -> list[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self.entries:
            raise KeyError(f"Tensor '{name}' not found in '{self.path}'")
        e = self.entries[name]
        _, tdtype, ndtype = _DTYPES[e.dtype]
        arr = np.frombuffer(self._map, dtype=ndtype, count=e.numel, offset=self._payload + e.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; nothing writes through the view
            t = torch.from_numpy(arr)
        if e.dtype == "BF16":
            t = t.view(torch.bfloat16)
        return t.reshape(e.shape)

    def close(self) -> None:
        # views handed out keep the map alive; closing is only safe once they are gone
        try:
            self._map.close()
        except BufferError:
            pass
        self._fh.close()


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """Write CPU tensors in the order given; offsets are laid out back to back."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).reshape(-1) if t.dtype != torch.bool else t.to(torch.uint8).reshape(-1)
        nbytes = raw.numel()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for raw in blobs:
            fh.write(raw.numpy().tobytes())


def list_weight_files(model_dir: str) -> list[str]:
    """All ``*.safetensors`` / ``*.safetensor`` files of a folder, sorted (demo/qwen3_infer.cpp:62-83)."""
    files = [os.path.join(model_dir, f) for f in sorted(os.listdir(model_dir))
             if f.endswith(".safetensors") or f.endswith(".safetensor")]
    return files
