"""Reading and writing safetensors files.

Layout: 8 bytes little-endian header length, a JSON header
`name -> {dtype, shape, data_offsets}`, then the raw little-endian data.  The
reference's container is GGUF (alpacca/gguf.py:82-194: mmap, tensor table
name -> shape, dtype, offset, zero-copy `tensor_bytes`); this is the same idea
for the other container: the file is mapped, the table is checked once, and a
tensor is a view of the mapping until it is copied to the device.
"""
from __future__ import annotations

import ctypes
import json
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
    """One mapped file; `tensors` is its table, `get(name)` a CPU view.

    The file is opened, mapped, parsed and checked by the native reader
    (`csrc/safetensors_reader.cpp`); this class is its Python face."""

    _lib = None

    @classmethod
    def _reader(cls):
        if cls._lib is None:
            from ..ops import build
            lib = build.load("safetensors_reader")
            lib.st_open.restype = ctypes.c_void_p
            lib.st_open.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]
            lib.st_count.argtypes = [ctypes.c_void_p]
            lib.st_entry.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_char_p),
                                     ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_longlong), ctypes.c_int,
                                     ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong)]
            lib.st_metadata_count.argtypes = [ctypes.c_void_p]
            lib.st_metadata.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_char_p),
                                        ctypes.POINTER(ctypes.c_char_p)]
            lib.st_data.restype = ctypes.c_void_p
            lib.st_data.argtypes = [ctypes.c_void_p]
            lib.st_data_len.restype = ctypes.c_longlong
            lib.st_data_len.argtypes = [ctypes.c_void_p]
            lib.st_close.argtypes = [ctypes.c_void_p]
            cls._lib = lib
        return cls._lib

    def __init__(self, path):
        self.path = Path(path)
        lib = self._reader()
        err = ctypes.create_string_buffer(512)
        self._handle = lib.st_open(str(self.path).encode(), err, len(err))
        if not self._handle:
            raise SafetensorsError(f"{self.path}: {err.value.decode(errors='replace')}")
        self.tensors: dict[str, TensorInfo] = {}
        name, dtype = ctypes.c_char_p(), ctypes.c_char_p()
        shape = (ctypes.c_longlong * 16)()
        lo, hi = ctypes.c_longlong(), ctypes.c_longlong()
        try:
            for i in range(lib.st_count(self._handle)):
                rank = lib.st_entry(self._handle, i, ctypes.byref(name), ctypes.byref(dtype), shape, 16,
                                    ctypes.byref(lo), ctypes.byref(hi))
                n, dt = name.value.decode(), dtype.value.decode()
                if rank > 16:
                    raise SafetensorsError(f"{self.path}: tensor {n} has {rank} dimensions")
                if dt not in DTYPES:
                    raise SafetensorsError(f"{self.path}: tensor {n} has unsupported dtype {dt}")
                self.tensors[n] = TensorInfo(n, dt, tuple(shape[d] for d in range(rank)), lo.value, hi.value)
            self.metadata = {}
            key, value = ctypes.c_char_p(), ctypes.c_char_p()
            for i in range(lib.st_metadata_count(self._handle)):
                lib.st_metadata(self._handle, i, ctypes.byref(key), ctypes.byref(value))
                self.metadata[key.value.decode()] = value.value.decode()
            self._data = lib.st_data(self._handle)
            self._data_len = lib.st_data_len(self._handle)
        except Exception:
            self.close()
            raise

    def get(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the tensor in its stored dtype (copy it before writing).  The view
        keeps the file mapped for as long as it lives."""
        if not self._handle:
            raise SafetensorsError(f"{self.path} is closed")
        ti = self.tensors[name]
        if ti.numel == 0:
            return torch.empty(ti.shape, dtype=DTYPES[ti.dtype])
        raw = (ctypes.c_ubyte * (ti.end - ti.begin)).from_address(self._data + ti.begin)
        with warnings.catch_warnings():   # the mapping is read-only; callers copy before writing
            warnings.simplefilter("ignore", UserWarning)
            t = torch.frombuffer(raw, dtype=DTYPES[ti.dtype], count=ti.numel)
        t = t.reshape(ti.shape)
        t._alpacca_file = self            # a view must not outlive the mapping
        self._views += 1
        return t

    _views = 0

    def close(self):
        """Unmaps the file, unless views of it were handed out: then the mapping lives as long as
        this object (which every view refers to)."""
        if self._handle and self._views == 0:
            self._reader().st_close(self._handle)
            self._handle = None

    def __del__(self):
        try:
            if getattr(self, "_handle", None):
                self._reader().st_close(self._handle)
                self._handle = None
        except Exception:
            pass


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
