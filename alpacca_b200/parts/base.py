"""Interfaces of the parts a decoder is put together from.

A part owns its sizes and constants (given to its constructor), the names and
shapes of its tensors in a checkpoint (`param_specs`), and its computation.  No
part knows which model it is in: it never reads a configuration object.

    Norm          forward(residual, delta, out=None, rows=None) -> normed activations
    Mixer         cache_spec() ; forward(h, ctx, cache, write_cache) -> delta
    FeedForward   forward(h, ctx) -> delta
    PositionEncoding  rotation tables for q/k and/or a term added to the embeddings
    Block         cache_specs() ; forward(stream, ctx, cache, write_cache): arranges the four above

`ctx` is the step's `StepContext` (device index tensors of the packed batch);
`cache` is what the mixer's `cache_spec()` asked for, for the cache entry that
the schedule gives this run of the layer: a `KVLayerView` or a `StateLayerView`.
A block says what its run keeps per sequence with `cache_specs()`, one spec for
each of its parts that keeps something; with one spec its `forward` gets that
entry's view, with several a list of views in the same order, with none `None`.

A norm without a kernel of its own (optional; steps of a few rows).  A norm whose
`deferred()` gives (weight, width, eps) is one factor per row, 1 / rms, times a weight per
column, so the product before it and the product after it can share its work.  A mixer or
feed-forward that sets `adds_to_residual` accepts `then=(residual, norm)`: it may add its output
to the residual itself and return an `OwedNorm` for `norm` instead of a delta (or a plain delta
when it cannot, e.g. for many rows).  One whose `accepts_owed_norm(n_rows)` says yes takes an
`OwedNorm` as its input `h` in a step of that many rows.  Parts that define neither never see
either; the block then runs the norm's own kernel.
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


@dataclass
class OwedNorm:
    """Rows whose RMS norm the reading product finishes: `x` holds residual * norm weight in the
    activation dtype, `ss` [rows, n_part] float32 partial sums of the residual's squares; every
    row still owes the division by sqrt(sum(ss[row]) / width + eps).  `norm` is the norm it
    stands for."""
    x: torch.Tensor
    ss: torch.Tensor
    width: int
    eps: float
    norm: object = None

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device


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

    def deferred(self):
        """(weight float32 [width], width, eps) if this norm is residual * weight / rms(residual)
        and may be finished by the product that reads it (see `OwedNorm`), else None."""
        return None


class Mixer(Part):
    #: `forward` accepts `then=(residual, norm)` (see the head of this file)
    adds_to_residual = False

    def accepts_owed_norm(self, n_rows: int) -> bool:
        """Whether `forward` takes an `OwedNorm` as `h` in a step of `n_rows` rows."""
        return False

    def cache_spec(self) -> KVSpec | StateSpec | None:
        return None

    def forward(self, h, ctx, cache, write_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    adds_to_residual = False

    def accepts_owed_norm(self, n_rows: int) -> bool:
        return False

    def forward(self, h, ctx):
        raise NotImplementedError


class Block(Part):
    """How a layer arranges its parts.  Anything with this `forward` serves as a block; one
    that has a single `.mixer` and does not define `cache_specs` is read as if it were this
    default."""

    def cache_specs(self) -> list:
        """What one run of this block keeps per sequence: a `KVSpec` or `StateSpec` for each part
        that keeps something, in the order in which `forward` wants their views."""
        mixer = getattr(self, "mixer", None)
        spec = mixer.cache_spec() if mixer is not None else None
        return [spec] if spec is not None else []

    def forward(self, stream, ctx, cache, write_cache: bool = True) -> None:
        raise NotImplementedError


def block_cache_specs(block) -> list:
    """`block.cache_specs()`, or for a block that does not define it, its `.mixer`'s spec."""
    own = getattr(block, "cache_specs", None)
    if own is not None:
        return [s for s in own() if s is not None]
    return Block.cache_specs(block)


class PositionEncoding(Part):
    """Default: no position information at all."""

    def rotation(self):
        """(cos, sin, n_rot, pairing code) for the rotation of q and k, or None."""
        return None

    def add_to_embeddings(self, residual, ctx) -> None:
        """Hook for encodings that add a term to the embedded tokens."""
