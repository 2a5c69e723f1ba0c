"""A small reader and writer for the safetensors file format.

A file is an 8-byte little-endian header length, a JSON header that maps each tensor name
to `{"dtype", "shape", "data_offsets": [begin, end]}` (offsets relative to the end of the
header), and the raw little-endian tensor bytes.  The reader maps the file and hands out
tensors by name without copying; the writer lays tensors out in name order, 8-byte aligned.
The reference reads the same files through the `safetensors` package (model/loader.py:57-60).
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Iterator

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """Read-only view of one .safetensors file."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: truncated (shorter than its 8-byte length field)")
        self._fh = open(self.path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: truncated (header of {hlen} bytes does not fit in {size})")
        try:
            header = json.loads(self._fh.read(hlen))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{self.path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + hlen
        self._entries: dict[str, tuple[torch.dtype, tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            dt = _DTYPES.get(info["dtype"])
            if dt is None:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {info['dtype']!r}")
            b, e = info["data_offsets"]
            shape = tuple(int(s) for s in info["shape"])
            n = 1
            for s in shape:
                n *= s
            if e - b != n * dt.itemsize or self._data_start + e > size:
                raise SafetensorsError(
                    f"{self.path}: tensor {name!r} {shape} {info['dtype']} does not match its byte range [{b}, {e})"
                    f" in a file of {size} bytes")
            self._entries[name] = (dt, shape, b, e)
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def keys(self) -> list[str]:
        return list(self._entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor's bytes as a (read-only, memory-mapped) CPU tensor."""
        dt, shape, b, e = self._entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable; it is only read
            flat = torch.frombuffer(self._mm, dtype=dt, count=(e - b) // dt.itemsize, offset=self._data_start + b)
        return flat.view(shape)

    def close(self) -> None:
        # tensors handed out keep the mapping alive through the buffer protocol
        self._fh.close()

    def __enter__(self) -> "SafetensorsFile":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r} has dtype {t.dtype}, which the format cannot hold")
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            fh.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def iter_model_files(folder: str | Path) -> Iterator[Path]:
    """Every *.safetensors file of a folder, sorted, as the reference reads them
    (model/loader.py:57)."""
    yield from sorted(Path(folder).glob("*.safetensors"))
