"""The gated feed-forward: a = silu(h Wg^T) * (h Wu^T); out = a Wd^T
(alpacca/model.py:510-514; SiLU on the gate, g/(1+exp(-g)), alpacca/tensor.py:150-160).

gate and up are held as one matrix, interleaved in groups of 8 rows, so that
one product feeds the activation kernel.
"""
from __future__ import annotations

from .base import BuildOptions, FeedForward
from .linear import Linear


class SwiGLU(FeedForward):
    def __init__(self, opts: BuildOptions, width: int, inner: int, prefix: str, bias: bool = False,
                 names=("gate_proj", "up_proj", "down_proj")):
        if inner % 8:
            raise ValueError(f"feed-forward width {inner} must be a multiple of 8 "
                             "(gate and up rows are interleaved in groups of 8)")
        self.opts, self.width, self.inner = opts, int(width), int(inner)
        g, u, d = names
        self.gate_up = Linear(opts, width, [(f"{prefix}.{g}", inner), (f"{prefix}.{u}", inner)], bias=bias,
                              interleave8=True)
        self.down = Linear(opts, inner, [(f"{prefix}.{d}", width)], bias=bias)

    adds_to_residual = True

    def accepts_owed_norm(self, n_rows: int) -> bool:
        return self.gate_up.accepts_owed_norm(n_rows)

    def forward(self, h, ctx, then=None):
        T = ctx.n_tokens
        act = self.gate_up.forward_swiglu(h, n_rows=T)
        return self.down.forward(act, n_rows=T, then=then)
