"""Read and write the safetensors container: 8 bytes of little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then the tensors' bytes.

Reading maps the file and hands out tensors by name without copying; nothing is converted
here. Only the element types a checkpoint of this engine can hold are known.
"""

from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path

import numpy as np
import torch

# safetensors name -> (torch dtype, numpy dtype the bytes are viewed as, bytes per element)
_TYPES = {
    "F32": (torch.float32, np.dtype("<f4"), 4),
    "BF16": (torch.bfloat16, np.dtype("<u2"), 2),
    "F16": (torch.float16, np.dtype("<f2"), 2),
    "F64": (torch.float64, np.dtype("<f8"), 8),
    "I32": (torch.int32, np.dtype("<i4"), 4),
    "I64": (torch.int64, np.dtype("<i8"), 8),
    "U8": (torch.uint8, np.dtype("u1"), 1),
    "BOOL": (torch.bool, np.dtype("u1"), 1),
}
_NAMES = {torch_dtype: name for name, (torch_dtype, _, _) in _TYPES.items()}


class SafetensorsFile:
    """One mapped file; `tensor(name)` views its bytes as a CPU tensor."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        with open(self.path, "rb") as handle:
            prefix = handle.read(8)
            if len(prefix) != 8:
                raise ValueError(f"{self.path}: not a safetensors file (too short)")
            (header_bytes,) = struct.unpack("<Q", prefix)
            size = self.path.stat().st_size
            if header_bytes > size - 8:
                raise ValueError(f"{self.path}: header length {header_bytes} exceeds the file")
            header = json.loads(handle.read(header_bytes))
            self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + header_bytes
        self.entries: dict[str, dict] = header
        for name, entry in header.items():
            if entry["dtype"] not in _TYPES:
                raise ValueError(f"{self.path}: tensor {name!r} has unsupported dtype {entry['dtype']}")
            begin, end = entry["data_offsets"]
            count = int(np.prod(entry["shape"], dtype=np.int64)) if entry["shape"] else 1
            if end - begin != count * _TYPES[entry["dtype"]][2] or self._base + end > size:
                raise ValueError(f"{self.path}: tensor {name!r} has inconsistent offsets")

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _TYPES[self.entries[name]["dtype"]][0]

    def tensor(self, name: str) -> torch.Tensor:
        entry = self.entries[name]
        torch_dtype, np_dtype, _ = _TYPES[entry["dtype"]]
        begin, end = entry["data_offsets"]
        flat = np.frombuffer(self._map, dtype=np_dtype, count=(end - begin) // np_dtype.itemsize,
                             offset=self._base + begin)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)  # the mapping is read-only; nothing writes to it
            tensor = torch.from_numpy(flat.copy() if flat.size == 0 else flat)
        if torch_dtype in (torch.bfloat16, torch.bool):
            tensor = tensor.view(torch_dtype)
        return tensor.reshape(entry["shape"])


def save_safetensors(tensors: dict[str, torch.Tensor], path: str | Path, metadata: dict | None = None) -> None:
    """Write CPU tensors by name, in name order, each aligned to 8 bytes by header padding."""
    header: dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise ValueError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    encoded = json.dumps(header, separators=(",", ":")).encode()
    encoded += b" " * (-(8 + len(encoded)) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(encoded)))
        handle.write(encoded)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.dtype in (torch.bfloat16,):
                t = t.view(torch.int16)
            elif t.dtype is torch.bool:
                t = t.view(torch.uint8)
            handle.write(t.numpy().tobytes())
