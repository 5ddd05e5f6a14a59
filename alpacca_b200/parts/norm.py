"""RMSNorm with a plain weight, fused with the residual add that precedes it.

inv = 1/sqrt(mean(x^2) + eps); y = (x * inv) * w  (alpacca/tensor.py:163-173);
the weight multiplies as it is (not 1 + w), eps is inside the root.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, Norm


class RMSNorm(Norm):
    def __init__(self, opts: BuildOptions, width: int, eps: float, name: str):
        self.opts, self.width, self.eps, self.name = opts, int(width), float(eps), name
        self.weight = None

    def own_param_specs(self):
        return [ParamSpec(f"{self.name}.weight", (self.width,), "vector", "one_plus_normal")]

    def load_own(self, fetch):
        self.weight = fetch(self.own_param_specs()[0])

    def deferred(self):
        if self.opts.dtype != torch.bfloat16 or self.weight is None:
            return None
        return self.weight, self.width, self.eps

    def forward(self, residual, delta, out=None, rows=None, n_rows=None):
        if out is None:
            n = (rows.numel() if rows is not None else residual.shape[0]) if n_rows is None else n_rows
            out = torch.empty((max(n, 0) if rows is not None else residual.shape[0], self.width),
                              dtype=self.opts.dtype, device=residual.device)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows=rows, n_rows=n_rows)
