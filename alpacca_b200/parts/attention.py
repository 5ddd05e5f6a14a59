"""Causal grouped-query attention over the paged cache.

q = h Wq^T, k = h Wk^T, v = h Wv^T (+ biases, added before the rotation:
alpacca/model.py:488-496); q, k rotated by position; k, v appended to the cache
before attending (:501-503); head h reads KV head h // (H/K) (:449,:459);
score = (q.k) * scale, keys up to the token's own position, softmax, weighted
sum of v (:447-467); output projection (:508).  The residual add is the block's.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import BuildOptions, KVSpec, Mixer, PositionEncoding
from .linear import Linear


class Attention(Mixer):
    def __init__(self, opts: BuildOptions, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: PositionEncoding | None, prefix: str, qkv_bias: bool = False, out_bias: bool = False,
                 window: int | None = None, scale: float | None = None,
                 names=("q_proj", "k_proj", "v_proj", "o_proj")):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} KV heads")
        if head_dim % 2:
            raise ValueError(f"head size {head_dim} must be even")
        self.opts = opts
        self.width, self.H, self.K, self.D = int(width), int(n_heads), int(n_kv_heads), int(head_dim)
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else self.D ** -0.5
        self.position = position
        q, k, v, o = names
        self.qkv = Linear(opts, width, [(f"{prefix}.{q}", self.H * self.D), (f"{prefix}.{k}", self.K * self.D),
                                        (f"{prefix}.{v}", self.K * self.D)], bias=qkv_bias)
        self.out = Linear(opts, self.H * self.D, [(f"{prefix}.{o}", width)], bias=out_bias)

    def cache_spec(self):
        return KVSpec(self.K, self.D, self.window)

    adds_to_residual = True

    def accepts_owed_norm(self, n_rows: int) -> bool:
        return self.qkv.accepts_owed_norm(n_rows)

    def forward(self, h, ctx, cache, write_cache: bool = True, then=None):
        T = ctx.n_tokens
        qkv = self.qkv.forward(h, n_rows=T)
        rot = self.position.rotation() if self.position is not None else None
        att = torch.empty((qkv.shape[0], self.H * self.D), dtype=qkv.dtype, device=qkv.device)
        ops.rope_attention(qkv, att, cache, ctx, self.H, self.K, self.D, self.scale, self.window or 0, rot,
                           write_cache=write_cache)
        # the attention kernel fills the SMs' shared memory, the product wants it as L1: it starts
        # when the attention has ended, not while it runs
        return self.out.forward(att, n_rows=T, start_early=False, then=then)
