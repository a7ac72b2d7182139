"""Reader and writer of the safetensors container.

Layout (src/safetensors.rs:42-98): ``<u64 little-endian header length><JSON header>
<raw tensor bytes>``; the header maps a tensor name to ``dtype``, ``shape`` and
``data_offsets`` (relative to the end of the header); ``__metadata__`` is skipped.
The reference reads F32, F16 and BF16 (src/safetensors.rs:66-76); this reader also
takes the integer types, for index tables.

Tensors are returned in their stored type, memory-mapped: nothing is widened here.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch


class SafeTensorsError(ValueError):
    pass


# name -> (torch dtype, numpy dtype used to view the bytes, bytes per element)
_DTYPES = {
    "F32": (torch.float32, np.dtype("<f4"), 4),
    "F16": (torch.float16, np.dtype("<f2"), 2),
    "BF16": (torch.bfloat16, np.dtype("<u2"), 2),
    "F64": (torch.float64, np.dtype("<f8"), 8),
    "I64": (torch.int64, np.dtype("<i8"), 8),
    "I32": (torch.int32, np.dtype("<i4"), 4),
    "I16": (torch.int16, np.dtype("<i2"), 2),
    "I8": (torch.int8, np.dtype("i1"), 1),
    "U8": (torch.uint8, np.dtype("u1"), 1),
    "BOOL": (torch.bool, np.dtype("u1"), 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorInfo:
    dtype: str
    shape: tuple[int, ...]
    start: int
    end: int

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]


class SafeTensorsFile:
    """An open weight file: ``names()``, ``info(name)``, ``tensor(name)``."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except OSError as e:
            raise SafeTensorsError(f"reading {self.path}: {e}") from e
        size = self.path.stat().st_size
        if size < 8:
            raise SafeTensorsError(f"{self.path}: file too small for a header length")
        (header_len,) = struct.unpack("<Q", self._fh.read(8))
        if header_len > size - 8:
            raise SafeTensorsError(f"{self.path}: header length exceeds file size")
        raw = self._fh.read(header_len)
        try:
            header = json.loads(raw.decode("utf-8"))
        except UnicodeDecodeError as e:
            raise SafeTensorsError(f"{self.path}: header is not UTF-8") from e
        except json.JSONDecodeError as e:
            raise SafeTensorsError(f"{self.path}: header JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafeTensorsError(f"{self.path}: header is not a JSON object")
        self._data_start = 8 + header_len
        data_len = size - self._data_start
        self.metadata = header.get("__metadata__") or {}
        self._infos: dict[str, TensorInfo] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype = info["dtype"]
                shape = tuple(int(s) for s in info["shape"])
                start, end = (int(o) for o in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as e:
                raise SafeTensorsError(f"{self.path}: {name}: bad header entry") from e
            if dtype not in _DTYPES:
                raise SafeTensorsError(
                    f"{self.path}: {name}: unsupported dtype {dtype} "
                    f"(this reader takes {sorted(_DTYPES)})")
            n = 1
            for s in shape:
                n *= s
            if end - start != n * _DTYPES[dtype][2] or start < 0 or end > data_len:
                raise SafeTensorsError(f"{self.path}: {name}: size mismatch")
            self._infos[name] = TensorInfo(dtype, shape, start, end)
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> list[str]:
        return sorted(self._infos)

    def __contains__(self, name: str) -> bool:
        return name in self._infos

    def info(self, name: str) -> TensorInfo:
        try:
            return self._infos[name]
        except KeyError:
            raise SafeTensorsError(f"missing tensor '{name}'") from None

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor in the stored dtype (a copy, so the file may be closed)."""
        info = self.info(name)
        tdtype, ndtype, _ = _DTYPES[info.dtype]
        buf = np.frombuffer(self._mm, dtype=ndtype, count=(info.end - info.start) // ndtype.itemsize,
                            offset=self._data_start + info.start)
        arr = np.array(buf, copy=True).reshape(info.shape)
        t = torch.from_numpy(arr)
        if tdtype is torch.bfloat16:
            t = t.view(torch.int16).view(torch.bfloat16)
        elif tdtype is torch.bool:
            t = t.to(torch.bool)
        return t

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor],
                      metadata: dict[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU or device, any supported dtype) in the given order."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs = []
    offset = 0
    for name, t in tensors.items():
        t = t.detach().to("cpu").contiguous()
        if t.dtype not in _NAMES:
            raise SafeTensorsError(f"{name}: cannot store dtype {t.dtype}")
        if t.dtype is torch.bfloat16:
            raw = t.view(torch.int16).numpy().tobytes()
        elif t.dtype is torch.bool:
            raw = t.to(torch.uint8).numpy().tobytes()
        else:
            raw = t.numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
