"""Reading and writing safetensors files.

Layout: 8 bytes little-endian header length, a JSON header
`name -> {dtype, shape, data_offsets}`, then the raw little-endian data.  The
reference's container is GGUF (alpacca/gguf.py:82-194: mmap, tensor table
name -> shape, dtype, offset, zero-copy `tensor_bytes`); this is the same idea
for the other container: the file is mapped, the table is checked once, and a
tensor is a view of the mapping until it is copied to the device.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from dataclasses import dataclass
from pathlib import Path

import torch

DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
DTYPE_NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple
    begin: int   # offsets from the start of the data section
    end: int

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class SafetensorsFile:
    """One mapped file; `tensors` is its table, `get(name)` a CPU view."""

    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        try:
            size = self.path.stat().st_size
            if size < 8:
                raise SafetensorsError(f"{self.path}: too short to be a safetensors file ({size} bytes)")
            (hlen,) = struct.unpack("<Q", self._f.read(8))
            if hlen > size - 8:
                raise SafetensorsError(f"{self.path}: header length {hlen} exceeds the file ({size} bytes)")
            try:
                header = json.loads(self._f.read(hlen).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{self.path}: header is not JSON: {e}") from None
            if not isinstance(header, dict):
                raise SafetensorsError(f"{self.path}: header must be a JSON object")
            self.data_start = 8 + hlen
            data_len = size - self.data_start
            self.metadata = header.pop("__metadata__", {}) or {}
            self.tensors: dict[str, TensorInfo] = {}
            for name, info in header.items():
                try:
                    dt, shape = info["dtype"], tuple(int(s) for s in info["shape"])
                    lo, hi = (int(x) for x in info["data_offsets"])
                except (KeyError, TypeError, ValueError):
                    raise SafetensorsError(f"{self.path}: malformed entry for tensor {name}") from None
                if dt not in DTYPES:
                    raise SafetensorsError(f"{self.path}: tensor {name} has unsupported dtype {dt}")
                ti = TensorInfo(name, dt, shape, lo, hi)
                want = ti.numel * DTYPES[dt].itemsize
                if lo < 0 or hi < lo or hi > data_len:
                    raise SafetensorsError(f"{self.path}: tensor {name} lies outside the file "
                                           f"(offsets {lo}..{hi}, data section {data_len} bytes)")
                if hi - lo != want:
                    raise SafetensorsError(f"{self.path}: tensor {name} of shape {list(shape)} {dt} "
                                           f"needs {want} bytes, has {hi - lo}")
                self.tensors[name] = ti
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        except Exception:
            self._f.close()
            raise

    def get(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the tensor in its stored dtype (copy it before writing)."""
        ti = self.tensors[name]
        if ti.numel == 0:
            return torch.empty(ti.shape, dtype=DTYPES[ti.dtype])
        with warnings.catch_warnings():   # the mapping is read-only; callers copy before writing
            warnings.simplefilter("ignore", UserWarning)
            t = torch.frombuffer(self._mm, dtype=DTYPES[ti.dtype], count=ti.numel,
                                 offset=self.data_start + ti.begin)
        return t.reshape(ti.shape)

    def close(self):
        # views handed out keep the mapping alive; closing only drops our handles
        self._mm = None
        self._f.close()


def write_safetensors(path, entries, metadata: dict | None = None) -> None:
    """Writes tensors one after another without holding them all.

    `entries`: list of (name, dtype name, shape, make) where `make()` returns
    the CPU tensor of that dtype and shape when its turn comes.
    """
    header, off = {}, 0
    for name, dt, shape, _ in entries:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * DTYPES[dt].itemsize
        header[name] = {"dtype": dt, "shape": [int(s) for s in shape], "data_offsets": [off, off + nbytes]}
        off += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name, dt, shape, make in entries:
            t = make()
            if t.dtype != DTYPES[dt] or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(f"tensor {name}: made {t.dtype} {tuple(t.shape)}, "
                                       f"declared {dt} {tuple(shape)}")
            t = t.detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
