"""How a layer arranges its parts: pre-norm, two residual adds
(x += Mixer(Norm1(x)); x += FeedForward(Norm2(x)), alpacca/model.py:486-514).

The residual stream is float32 in memory in both precisions.  A sub-layer's
output is not added at once: it waits in `stream.delta` and is added by the
next norm's fused kernel (which reads the stream anyway).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import FeedForward, Mixer, Norm, Part


@dataclass
class HiddenStream:
    residual: torch.Tensor            # float32 [T, E]
    delta: torch.Tensor | None = None  # output of the last sub-layer, not yet added


class PreNormBlock(Part):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm | None, ffn: FeedForward | None):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn

    def forward(self, stream: HiddenStream, ctx, cache, write_cache: bool = True) -> None:
        h = self.norm1.forward(stream.residual, stream.delta)
        stream.delta = self.mixer.forward(h, ctx, cache, write_cache)
        if self.ffn is not None:
            h = self.norm2.forward(stream.residual, stream.delta)
            stream.delta = self.ffn.forward(h, ctx)
