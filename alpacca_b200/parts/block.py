"""How a layer arranges its parts: pre-norm, two residual adds
(x += Mixer(Norm1(x)); x += FeedForward(Norm2(x)), alpacca/model.py:486-514).

The residual stream is float32 in memory in both precisions.  A sub-layer's
output is not added at once: it waits in `stream.delta` and is added by the
next norm's fused kernel (which reads the stream anyway).  In steps of a few
rows the norm has no kernel at all where the parts on both sides can share its
work (`OwedNorm` in base.py): the sub-layer adds its output to the residual
itself and hands `stream.owed` to the next reader.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import Block, FeedForward, Mixer, Norm, OwedNorm


@dataclass
class HiddenStream:
    residual: torch.Tensor            # float32 [T, E]
    delta: torch.Tensor | None = None  # output of the last sub-layer, not yet added
    owed: OwedNorm | None = None       # or: the residual is up to date and these rows stand for `owed.norm`
    next_norm: Norm | None = None      # set by the model: the norm that reads the stream after this block,
                                       # if its reader accepts an OwedNorm in this step


class PreNormBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm | None, ffn: FeedForward | None):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn

    def first_norm(self, n_rows: int) -> Norm | None:
        """The norm that reads the stream when this block starts, if in a step of `n_rows` rows the
        block accepts an `OwedNorm` for it from whatever ran before."""
        if _accepts(self.mixer, n_rows) and self.norm1.deferred() is not None:
            return self.norm1
        return None

    def forward(self, stream: HiddenStream, ctx, cache, write_cache: bool = True) -> None:
        next_norm, stream.next_norm = stream.next_norm, None
        h = _normed(self.norm1, stream)
        if self.ffn is None:
            _sublayer(stream, next_norm, self.mixer, h, ctx, cache, write_cache)
            return
        after_mixer = self.norm2 if _accepts(self.ffn, ctx.n_tokens) else None
        _sublayer(stream, after_mixer, self.mixer, h, ctx, cache, write_cache)
        h = _normed(self.norm2, stream)
        _sublayer(stream, next_norm, self.ffn, h, ctx)


def _accepts(part, n_rows: int) -> bool:
    accepts = getattr(part, "accepts_owed_norm", None)
    return bool(accepts(n_rows)) if accepts is not None else False


def _normed(norm: Norm, stream: HiddenStream):
    """What `norm` gives its reader: the rows prepared for it, or its own kernel's output."""
    if stream.owed is not None:
        owed, stream.owed = stream.owed, None
        if owed.norm is not norm:
            raise RuntimeError("rows were prepared for another norm than the one that reads them")
        return owed
    return norm.forward(stream.residual, stream.delta)


def _sublayer(stream: HiddenStream, then_norm: Norm | None, part, h, *args) -> None:
    """Runs a mixer or feed-forward; its output waits in `stream.delta`, or, where the part and the
    norm after it allow, is added by the part itself and prepared for that norm (`stream.owed`)."""
    if (then_norm is not None and getattr(part, "adds_to_residual", False)
            and then_norm.deferred() is not None):
        out = part.forward(h, *args, then=(stream.residual, then_norm))
    else:
        out = part.forward(h, *args)
    if isinstance(out, OwedNorm):
        stream.owed, stream.delta = out, None
    else:
        stream.delta = out
