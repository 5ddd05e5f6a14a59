"""The matrix product y = x @ W^T (+ b), W stored [out, in] as in the checkpoint.

Several checkpoint matrices that read the same input can be held as one fused
matrix (q|k|v, gate|up).  In the 32-bit path the product is the package's own
FMA kernel; in the bfloat16 path it is the skinny-matrix kernel for the few rows
of a decode step and the library matrix product otherwise (the reference uses
BLAS for every product: alpacca/tensor.py:82-97).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, OwedNorm, Part


class Linear(Part):
    def __init__(self, opts: BuildOptions, in_features: int, sources, bias: bool = False,
                 interleave8: bool = False, out_dtype: torch.dtype | None = None):
        """`sources`: list of (checkpoint prefix, rows); tensors `<prefix>.weight`
        [rows, in] (and `<prefix>.bias` [rows]) are stacked in that order.
        `interleave8`: two sources of equal size are interleaved in groups of 8
        rows (8 of the first, 8 of the second, ...), the layout `ops.swiglu` reads.
        `out_dtype` float32 gives float32 results from bfloat16 inputs (logits)."""
        self.opts = opts
        self.in_features = int(in_features)
        self.sources = [(p, int(r)) for p, r in sources]
        self.out_features = sum(r for _, r in self.sources)
        self.has_bias = bool(bias)
        self.interleave8 = bool(interleave8)
        self.out_dtype = out_dtype or opts.dtype
        if interleave8:
            if len(self.sources) != 2 or self.sources[0][1] != self.sources[1][1] or self.sources[0][1] % 8:
                raise ValueError("interleave8 needs two sources of equal size, a multiple of 8 rows "
                                 f"(got {[r for _, r in self.sources]})")
        self.weight = None
        self.bias = None

    def own_param_specs(self):
        specs = [ParamSpec(f"{p}.weight", (r, self.in_features), "matrix", "normal") for p, r in self.sources]
        if self.has_bias:
            specs += [ParamSpec(f"{p}.bias", (r,), "vector", "normal") for p, r in self.sources]
        return specs

    def _stack(self, tensors):
        if len(tensors) == 1:
            return tensors[0]
        if self.interleave8:
            a, b = tensors
            tail = a.shape[1:]
            return torch.cat([a.reshape(-1, 8, *tail), b.reshape(-1, 8, *tail)], dim=1).reshape(-1, *tail).contiguous()
        return torch.cat(tensors, dim=0).contiguous()

    def load_own(self, fetch):
        self.weight = self._stack([fetch(ParamSpec(f"{p}.weight", (r, self.in_features), "matrix"))
                                   for p, r in self.sources])
        if self.has_bias:
            self.bias = self._stack([fetch(ParamSpec(f"{p}.bias", (r,), "vector")) for p, r in self.sources])

    def share_weight(self, tensor: torch.Tensor):
        """Uses an existing tensor as the matrix (a tied head)."""
        self.weight = tensor

    def accepts_owed_norm(self, n_rows: int) -> bool:
        """Whether `forward` should be given an `OwedNorm` in a step of `n_rows` rows (it can take one
        whenever the skinny product runs; it pays only for some shapes, see `ops.owed_norm_pays`)."""
        return (self.opts.dtype == torch.bfloat16 and self.weight is not None
                and ops.owed_norm_pays(n_rows, self.out_features, self.in_features, self.weight.device))

    def forward(self, x, n_rows: int | None = None, start_early: bool = True, then=None):
        """`start_early` off: the product's kernel may not start before the kernel before it has ended
        (see `ops.gemv_bf16`).  `x` may be an `OwedNorm` (the division by the rms is applied to the
        sums).  `then` = (residual, norm): where the step has few enough rows, the result is added to
        the residual here and an `OwedNorm` for `norm` is returned instead of the result."""
        n = x.shape[0] if n_rows is None else n_rows
        owed = None
        if isinstance(x, OwedNorm):
            owed, x = (x.ss, x.width, x.eps), x.x
        if then is not None and x.dtype == torch.bfloat16 and self.out_dtype == torch.bfloat16:
            residual, norm = then
            d = norm.deferred()
            if (d is not None and d[1] == self.out_features and ops.defers_norm(n, self.out_features)
                    and self.in_features % 8 == 0):
                out = torch.empty((x.shape[0], self.out_features), dtype=torch.bfloat16, device=x.device)
                _, ss = ops.gemv_bf16(x, self.weight, out, bias=self.bias, n_rows=n, start_early=start_early,
                                      owed=owed, residual=residual, norm_weight=d[0])
                return OwedNorm(out, ss, d[1], d[2], norm)
        out = torch.empty((x.shape[0], self.out_features), dtype=self.out_dtype, device=x.device)
        if x.dtype == torch.float32:
            ops.gemm_f32(x, self.weight, out, bias=self.bias, n_rows=n)
            return out
        return ops.linear_bf16(x, self.weight, out, n_rows=n, bias=self.bias, start_early=start_early, owed=owed)

    def forward_swiglu(self, x, n_rows: int | None = None) -> torch.Tensor:
        """silu(gate) * up of the interleaved gate|up product, [M, out_features / 2]."""
        n = x.shape[0] if n_rows is None else n_rows
        if isinstance(x, OwedNorm):
            act = torch.empty((x.shape[0], self.out_features // 2), dtype=x.dtype, device=x.device)
            return ops.gemv_bf16(x.x, self.weight, act, bias=self.bias, n_rows=n, swiglu=True,
                                 owed=(x.ss, x.width, x.eps))
        act = torch.empty((x.shape[0], self.out_features // 2), dtype=x.dtype, device=x.device)
        if x.dtype == torch.bfloat16 and self.in_features % 8 == 0:
            if n <= ops.GEMV_MAX_ROWS:
                return ops.gemv_bf16(x, self.weight, act, bias=self.bias, n_rows=n, swiglu=True)
            if n >= ops.TC_PERSISTENT_MIN_ROWS:
                # long prompts: the persistent tcgen05 product with the activation in its tail
                return ops.gemm_tc(x, self.weight, act, bias=self.bias, n_rows=n, swiglu=True, swap=False)
        return ops.swiglu(self.forward(x, n_rows=n), act, n_rows=n)
