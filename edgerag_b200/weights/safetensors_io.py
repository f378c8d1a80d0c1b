"""Reading and writing the safetensors container, by tensor name.

The format is an 8-byte little-endian header length, a JSON header mapping each name to
``{"dtype", "shape", "data_offsets"}``, then the raw little-endian tensor bytes.  The file is
memory-mapped, so a tensor's bytes are only touched when it is asked for.
"""

from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path

import numpy as np
import torch

_DTYPES: dict[str, tuple[torch.dtype, int]] = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


class SafetensorsFile:
    """A read-only view of one ``.safetensors`` file."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        if not self.path.is_file():
            raise SafetensorsError(f"{self.path} does not exist")
        self._file = open(self.path, "rb")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short for a header")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(f"{self.path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._file.read(header_len))
        except (json.JSONDecodeError, UnicodeDecodeError) as exc:
            raise SafetensorsError(f"{self.path}: header is not JSON ({exc})") from exc
        self.metadata = header.pop("__metadata__", {})
        self._data_start = 8 + header_len
        self._mmap = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries: dict[str, dict] = {}
        for name, info in header.items():
            code = info.get("dtype")
            if code not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name} has unknown dtype {code}")
            begin, end = info["data_offsets"]
            count = int(np.prod(info["shape"], dtype=np.int64)) if info["shape"] else 1
            if end - begin != count * _DTYPES[code][1] or self._data_start + end > size:
                raise SafetensorsError(f"{self.path}: tensor {name} has inconsistent offsets")
            self.entries[name] = info

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]][0]

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor as stored (a view of the mapping: copy or cast before the file is closed)."""
        info = self.entries[name]
        dtype, _ = _DTYPES[info["dtype"]]
        begin, end = info["data_offsets"]
        raw = np.frombuffer(self._mmap, dtype=np.uint8, count=end - begin, offset=self._data_start + begin)
        with warnings.catch_warnings():
            warnings.filterwarnings("ignore", message=".*not writable.*")
            flat = torch.from_numpy(raw)  # read-only memory: callers copy or cast, never write
        return flat.view(dtype).reshape(info["shape"])

    def close(self) -> None:
        try:
            self._mmap.close()
        except BufferError:
            pass  # a view is still alive; the mapping goes when it does
        self._file.close()

    def __enter__(self) -> "SafetensorsFile":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) to ``path`` in name order."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-(8 + len(blob)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
