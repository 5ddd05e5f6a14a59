"""Where tensors come from: a model folder, or a seed.

A source answers two questions: which tensors it has (`table()`: name ->
(dtype name, shape)) and what a tensor holds (`get(name)`: a tensor in its
stored dtype).  The loader works on this interface alone.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .safetensors_file import DTYPE_NAMES, DTYPES, SafetensorsError, SafetensorsFile


class FolderSource:
    """`model.safetensors`, or the shards that `model.safetensors.index.json` names."""

    def __init__(self, model_dir):
        self.model_dir = Path(model_dir)
        index = self.model_dir / "model.safetensors.index.json"
        single = self.model_dir / "model.safetensors"
        self.files: list[SafetensorsFile] = []
        self._where: dict[str, SafetensorsFile] = {}
        if single.is_file():
            shard_names = [single.name]
        elif index.is_file():
            weight_map = json.loads(index.read_text()).get("weight_map", {})
            shard_names = sorted(set(weight_map.values()))
            if not shard_names:
                raise SafetensorsError(f"{index} names no shards")
        else:
            raise SafetensorsError(f"no model.safetensors (or model.safetensors.index.json) in {self.model_dir}")
        for sn in shard_names:
            p = self.model_dir / sn
            if not p.is_file():
                raise SafetensorsError(f"shard {sn} named by the index is missing in {self.model_dir}")
            f = SafetensorsFile(p)
            self.files.append(f)
            for name in f.tensors:
                if name in self._where:
                    raise SafetensorsError(f"tensor {name} is in both {self._where[name].path.name} and {sn}")
                self._where[name] = f

    def table(self) -> dict[str, tuple[str, tuple]]:
        return {n: (f.tensors[n].dtype, f.tensors[n].shape) for n, f in self._where.items()}

    def get(self, name: str) -> torch.Tensor:
        return self._where[name].get(name)

    def close(self):
        for f in self.files:
            f.close()


def _name_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


class RandomSource:
    """Tensors drawn from a seed, each from a generator keyed by (seed, name), so
    that a tensor's values do not depend on which others were made before it.

    Matrices, embeddings and biases are N(0, std); norm weights 1 + N(0, std);
    values are drawn in float32 and then rounded to the storage dtype.  (The
    reference's own random models: tests/make_tiny_model.py:81-85,
    tests/make_bench_model.py:111-124, with norm weights of exactly 1.)
    """

    def __init__(self, param_specs, seed: int, dtype: torch.dtype = torch.bfloat16,
                 std: float = 0.02, device: str = "cpu"):
        self.specs = {s.name: s for s in param_specs if not s.absent}
        self.seed, self.dtype, self.std, self.device = int(seed), dtype, float(std), device

    def _stored_dtype(self, spec) -> torch.dtype:
        if spec.role == "int":
            return torch.int32
        return self.dtype

    def table(self):
        return {n: (DTYPE_NAMES[self._stored_dtype(s)], tuple(s.shape)) for n, s in self.specs.items()}

    def get(self, name: str) -> torch.Tensor:
        spec = self.specs[name]
        g = torch.Generator(device=self.device)
        g.manual_seed(_name_seed(self.seed, name))
        if spec.role == "int":
            return torch.zeros(spec.shape, dtype=torch.int32, device=self.device)
        if spec.init == "zeros":
            t = torch.zeros(spec.shape, dtype=torch.float32, device=self.device)
        else:
            t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=self.device) * self.std
            if spec.init == "one_plus_normal":
                t += 1.0
        return t.to(self._stored_dtype(spec))

    def close(self):
        pass


__all__ = ["FolderSource", "RandomSource", "DTYPES", "DTYPE_NAMES"]
