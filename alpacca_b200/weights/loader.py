"""Loading by tensor name.

The model says which tensors it expects (`ParamSpec`: name, shape, role); the
source says which it has.  Both lists are compared in full before anything is
copied, and every fault goes into one error: missing tensors, unexpected ones,
wrong shapes.  (The reference checks name by name and element counts only:
alpacca/model.py:258-291.)

In memory: a matrix is kept in the compute dtype (bfloat16 in the bfloat16
path: nothing is widened; float32 in the 32-bit path); small vectors that enter
32-bit arithmetic (norm weights, biases) are kept in float32, whatever they
were stored in; integer tables are int32; a tensor whose spec has role "keep32"
stays in 32-bit if it was stored so.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


class WeightError(ValueError):
    """Names and shapes of the source do not fit the model; lists every fault."""


@dataclass(frozen=True)
class ParamSpec:
    name: str                 # full tensor name in the checkpoint
    shape: tuple
    role: str = "matrix"      # "matrix" | "vector" | "int" | "keep32"
    init: str = "normal"      # random-weights mode: "normal" | "one_plus_normal" | "zeros"
    absent: bool = False      # declared but not stored (a tied head): must NOT be in the source


def check_names(specs, table: dict, where: str = "") -> None:
    missing, wrong, clash = [], [], []
    expected = {}
    for s in specs:
        if s.name in expected and not s.absent and not expected[s.name].absent:
            if tuple(expected[s.name].shape) != tuple(s.shape):
                clash.append(s.name)
            continue
        expected[s.name] = s
    for name, s in expected.items():
        if s.absent:
            continue
        if name not in table:
            missing.append(f"{name} {list(s.shape)}")
        elif tuple(table[name][1]) != tuple(s.shape):
            wrong.append(f"{name}: expected {list(s.shape)}, found {list(table[name][1])}")
    unexpected = [f"{n} {list(table[n][1])}" for n in table
                  if n not in expected or expected[n].absent]
    if missing or wrong or unexpected or clash:
        parts = []
        if missing:
            parts.append(f"{len(missing)} missing: " + ", ".join(missing))
        if unexpected:
            parts.append(f"{len(unexpected)} unexpected: " + ", ".join(unexpected))
        if wrong:
            parts.append(f"{len(wrong)} of wrong shape: " + "; ".join(wrong))
        if clash:
            parts.append("declared twice with different shapes: " + ", ".join(clash))
        raise WeightError(f"weights{' in ' + where if where else ''} do not fit the model — " + " | ".join(parts))


class Fetcher:
    """Hands tensors to the parts: `fetch(spec)` returns the tensor on the device
    in the dtype that its role asks for."""

    def __init__(self, source, device, compute_dtype: torch.dtype):
        self.source, self.device, self.compute_dtype = source, device, compute_dtype
        self.bytes_loaded = 0

    def __call__(self, spec: ParamSpec) -> torch.Tensor:
        t = self.source.get(spec.name)
        if spec.role == "int":
            if t.dtype.is_floating_point:
                raise WeightError(f"tensor {spec.name} must hold integers, is {t.dtype}")
            out = t.to(device=self.device, dtype=torch.int32)
        elif spec.role == "vector":
            out = t.to(device=self.device).to(torch.float32)
        elif spec.role == "keep32":
            keep = t.dtype == torch.float32
            out = t.to(device=self.device).to(torch.float32 if keep else self.compute_dtype)
        else:
            if not t.dtype.is_floating_point:
                raise WeightError(f"tensor {spec.name} must hold floating-point values, is {t.dtype}")
            out = t.to(device=self.device).to(self.compute_dtype)
        out = out.contiguous()
        if out.data_ptr() == t.data_ptr():   # never hand out a view of the mapped file
            out = out.clone()
        self.bytes_loaded += out.numel() * out.element_size()
        return out
