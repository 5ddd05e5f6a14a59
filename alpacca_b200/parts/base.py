"""Interfaces of the parts a decoder is put together from.

A part owns its sizes and constants (given to its constructor), the names and
shapes of its tensors in a checkpoint (`param_specs`), and its computation.  No
part knows which model it is in: it never reads a configuration object.

    Norm          forward(residual, delta, out=None, rows=None) -> normed activations
    Mixer         cache_spec() ; forward(h, ctx, cache, write_cache) -> delta
    FeedForward   forward(h, ctx) -> delta
    PositionEncoding  rotation tables for q/k and/or a term added to the embeddings
    Block         forward(stream, ctx, cache, write_cache): arranges the four above

`ctx` is the step's `StepContext` (device index tensors of the packed batch);
`cache` is what the mixer's `cache_spec()` asked for, for the cache entry that
the schedule gives this run of the layer: a `KVLayerView` or a `StateLayerView`.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..weights.loader import ParamSpec


@dataclass(frozen=True)
class BuildOptions:
    """What a part needs to know about where and in which precision it runs."""
    dtype: torch.dtype = torch.bfloat16        # activations, matrices, cache
    device: str | torch.device = "cuda"
    max_positions: int = 4096                  # longest sequence the engine will hold


@dataclass(frozen=True)
class KVSpec:
    """The mixer keeps keys and values of `n_kv_heads` x `head_dim` per token;
    `window` = how many of the latest keys it reads (None: all)."""
    n_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateSpec:
    """The mixer keeps a state of fixed shape per sequence (zero at a sequence's start)."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts: parameters by checkpoint name, loading, sub-parts."""

    #: whether `forward` only launches work on the current stream, from device
    #: data alone (no host reads of tensors, no shapes that depend on values),
    #: so that a decode step may be captured in a CUDA graph
    graph_capturable = True

    def children(self) -> list["Part"]:
        return [v for v in vars(self).values() if isinstance(v, Part)] + \
               [p for v in vars(self).values() if isinstance(v, (list, tuple)) for p in v if isinstance(p, Part)]

    def own_param_specs(self) -> list[ParamSpec]:
        return []

    def param_specs(self) -> list[ParamSpec]:
        out = list(self.own_param_specs())
        for c in self.children():
            out.extend(c.param_specs())
        return out

    def load_own(self, fetch) -> None:
        pass

    def load(self, fetch) -> None:
        """`fetch(ParamSpec)` returns the tensor on the device in the dtype of its role."""
        self.load_own(fetch)
        for c in self.children():
            c.load(fetch)

    def all_capturable(self) -> bool:
        return self.graph_capturable and all(c.all_capturable() for c in self.children())


class Norm(Part):
    def forward(self, residual, delta, out=None, rows=None, n_rows=None):
        """normed(residual + delta); adds delta into the residual unless `rows` picks rows."""
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self) -> KVSpec | StateSpec | None:
        return None

    def forward(self, h, ctx, cache, write_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h, ctx):
        raise NotImplementedError


class PositionEncoding(Part):
    """Default: no position information at all."""

    def rotation(self):
        """(cos, sin, n_rot, pairing code) for the rotation of q and k, or None."""
        return None

    def add_to_embeddings(self, residual, ctx) -> None:
        """Hook for encodings that add a term to the embedded tokens."""
