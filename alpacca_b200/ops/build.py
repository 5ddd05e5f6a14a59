"""Compiles the CUDA sources of `csrc/` for sm_100a, one shared library per
source file, when a library is first needed.

Libraries are plain `extern "C"` entry points loaded with ctypes; they are kept
beside the sources (`csrc/_build/`) when that folder can be written, else in a
per-user folder under the temporary directory.  A library is rebuilt when its
source, a header it can include, or the compiler flags change.  While nvcc runs
a line is printed now and then, so that a first call is not mistaken for a hang.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC"]

_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _find_nvcc() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").is_file():
            return str(Path(cand) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc was not found (looked in $CUDA_HOME, /usr/local/cuda and PATH); "
                     "the CUDA kernels of alpacca_b200 cannot be built")


_chosen_dir: Path | None = None


def _build_dir() -> Path:
    global _chosen_dir
    if _chosen_dir is not None:
        return _chosen_dir
    override = os.environ.get("ALPACCA_B200_BUILD_DIR")
    cands = [Path(override)] if override else []
    cands.append(CSRC / "_build")
    cands.append(Path(tempfile.gettempdir()) / f"alpacca_b200-build-{os.getuid()}")
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            with tempfile.NamedTemporaryFile(dir=d, prefix=".probe"):
                pass
            _chosen_dir = d
            return d
        except OSError:
            continue
    raise BuildError(f"no writable folder for built libraries (tried {', '.join(map(str, cands))})")


def _fingerprint(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.name.encode())
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _say(msg: str) -> None:
    print(f"[alpacca_b200] {msg}", file=sys.stderr, flush=True)


def _compile(cmd: list[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"still building {what} ({time.time() - t0:.0f} s)")
    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"building {what} failed:\n$ {' '.join(cmd)}\n{out}")
    _say(f"built {what} in {time.time() - t0:.1f} s")


def library_path(name: str) -> Path:
    """Builds `csrc/<name>.cu` (or `.cpp`) if needed and returns the library's path."""
    src = CSRC / f"{name}.cu"
    is_cuda = src.is_file()
    if not is_cuda:
        src = CSRC / f"{name}.cpp"
        if not src.is_file():
            raise BuildError(f"no source for library {name!r} in {CSRC}")
    flags = NVCC_FLAGS if is_cuda else HOST_FLAGS
    fp = _fingerprint(src, flags)
    out_dir = _build_dir()
    lib = out_dir / f"lib{name}.so"
    stamp = out_dir / f"lib{name}.stamp"
    if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == fp:
        return lib
    tmp = out_dir / f"lib{name}.{os.getpid()}.{threading.get_ident()}.tmp.so"
    if is_cuda:
        cmd = [_find_nvcc(), *flags, "-I", str(CSRC), "-o", str(tmp), str(src)]
    else:
        cmd = [os.environ.get("CXX", "g++"), *flags, "-I", str(CSRC), "-o", str(tmp), str(src)]
    _say(f"building {src.name} for sm_100a ..." if is_cuda else f"building {src.name} ...")
    try:
        _compile(cmd, src.name)
        os.replace(tmp, lib)
        stamp.write_text(fp)
    finally:
        if tmp.exists():
            tmp.unlink()
    return lib


def load(name: str) -> ctypes.CDLL:
    """The loaded library `name`, building it first when needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(str(library_path(name)))
            _loaded[name] = lib
        return lib


ALL_LIBRARIES = ("elementwise", "attention_simt", "attention_mma", "gemm_f32", "gemv_bf16", "gemm_tc", "attention_tc", "attention_stream", "sampling", "safetensors_reader")


def build_all(names=ALL_LIBRARIES) -> list[Path]:
    """Builds every library (in parallel); used by the build check and by installers."""
    results: dict[str, object] = {}

    def work(n):
        try:
            results[n] = library_path(n)
        except Exception as e:  # noqa: BLE001 - reported below
            results[n] = e
    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    errors = [str(v) for v in results.values() if isinstance(v, Exception)]
    if errors:
        raise BuildError("\n".join(errors))
    return [results[n] for n in names]
