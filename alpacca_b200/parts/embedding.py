"""Token embedding (row gather, no scaling: alpacca/model.py:482) and the
vocabulary head (logits = W . norm(x), alpacca/model.py:518; tied: the head is
the embedding table itself, :320-322).  Logits are float32 in both precisions.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, Part
from .linear import Linear


class TokenEmbedding(Part):
    def __init__(self, opts: BuildOptions, vocab: int, width: int, name: str):
        self.opts, self.vocab, self.width, self.name = opts, int(vocab), int(width), name
        self.weight = None

    def own_param_specs(self):
        return [ParamSpec(f"{self.name}.weight", (self.vocab, self.width), "matrix", "normal")]

    def load_own(self, fetch):
        self.weight = fetch(self.own_param_specs()[0])

    def forward(self, tokens: torch.Tensor, n_rows: int) -> torch.Tensor:
        out = torch.empty((n_rows, self.width), dtype=torch.float32, device=tokens.device)
        return ops.embed_rows(self.weight, tokens[:n_rows], out)


class VocabHead(Part):
    def __init__(self, opts: BuildOptions, vocab: int, width: int, name: str,
                 tied_to: TokenEmbedding | None = None):
        self.opts, self.vocab, self.width, self.name = opts, int(vocab), int(width), name
        self.tied_to = tied_to
        self.proj = Linear(opts, width, [(name, vocab)], out_dtype=torch.float32)

    def children(self):
        return [] if self.tied_to is not None else [self.proj]

    def own_param_specs(self):
        if self.tied_to is not None:   # declared so that a stray stored head is reported, not ignored
            return [ParamSpec(f"{self.name}.weight", (self.vocab, self.width), "matrix", absent=True)]
        return []

    def load_own(self, fetch):
        pass

    def forward(self, h: torch.Tensor, n_rows: int | None = None) -> torch.Tensor:
        if self.tied_to is not None and self.proj.weight is not self.tied_to.weight:
            self.proj.share_weight(self.tied_to.weight)
        return self.proj.forward(h, n_rows=n_rows)
