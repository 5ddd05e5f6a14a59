"""A decoder as data: its parts and the order in which they run.

`DecoderSpec` is what an architecture's build function returns: the embedding,
the layers (each a block of parts), the schedule, the final norm and the head.
The schedule is a list of runs; a run names the layer it executes and the cache
entries it uses.  Naming a layer in two runs executes it twice (each run with
cache entries of its own); a run whose `reads_entry_of` names an earlier run
reads that run's cache and writes none.  What a run keeps is the block's to say
(`cache_specs()`): one entry for each of its parts that keeps keys and values or
a state, none for a block that keeps nothing.

`DecoderModel` executes a spec for one step: embed the step's tokens, run the
schedule, norm the wanted rows, project them to logits
(alpacca/model.py:469-518 is the reference's form of the same pass).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import BuildOptions, Norm, Part, PositionEncoding, block_cache_specs
from ..parts.block import HiddenStream
from ..parts.embedding import TokenEmbedding, VocabHead
from ..weights.loader import Fetcher, check_names


@dataclass(frozen=True)
class Run:
    layer: int                       # index into DecoderSpec.layers
    reads_entry_of: int | None = None  # index of an earlier run whose cache this run reads


@dataclass
class DecoderSpec:
    embedding: TokenEmbedding
    layers: list                     # blocks: forward(stream, ctx, cache, write_cache)
    final_norm: Norm
    head: VocabHead
    schedule: list[Run] = field(default_factory=list)
    position: PositionEncoding | None = None   # an encoding that adds to the embeddings, if any
    stop_token_ids: tuple = ()
    vocab_size: int = 0

    def __post_init__(self):
        if not self.schedule:
            self.schedule = [Run(i) for i in range(len(self.layers))]
        for i, r in enumerate(self.schedule):
            if not 0 <= r.layer < len(self.layers):
                raise ValueError(f"run {i} names layer {r.layer}, the model has {len(self.layers)}")
            if r.reads_entry_of is not None:
                if not 0 <= r.reads_entry_of < i or self.schedule[r.reads_entry_of].reads_entry_of is not None:
                    raise ValueError(f"run {i} must read the cache of an earlier run that owns one")
        if not self.vocab_size:
            self.vocab_size = self.head.vocab


class DecoderModel(Part):
    def __init__(self, spec: DecoderSpec, opts: BuildOptions, config=None):
        self.spec, self.opts, self.config = spec, opts, config
        # the cache entries of each run: its own (one for each spec of its block), or those of the
        # run it reads
        self._entry_specs: list = []
        self.entries_of_run: list[list[int]] = []
        for i, r in enumerate(spec.schedule):
            if r.reads_entry_of is not None:
                theirs = self.entries_of_run[r.reads_entry_of]
                mine = block_cache_specs(spec.layers[r.layer])
                if [self._entry_specs[e] for e in theirs] != mine:
                    raise ValueError(f"run {i} reads the cache of run {r.reads_entry_of}, which keeps "
                                     "something else than this run's layer would")
                self.entries_of_run.append(theirs)
                continue
            specs = block_cache_specs(spec.layers[r.layer])
            self.entries_of_run.append(list(range(len(self._entry_specs), len(self._entry_specs) + len(specs))))
            self._entry_specs.extend(specs)

    def children(self):
        s = self.spec
        out = [s.embedding, *s.layers, s.final_norm, s.head]
        if s.position is not None:
            out.append(s.position)
        return out

    def cache_entry_specs(self):
        """The spec of every cache entry of the schedule, in the order of `entries_of_run`."""
        return list(self._entry_specs)

    def _views(self, i: int, cache, block_tables):
        """What run `i`'s block gets as `cache`: its entry's view, a list of views, or None."""
        views = [cache.entry_view(e, block_tables) for e in self.entries_of_run[i]]
        return views[0] if len(views) == 1 else (views or None)

    def load_weights(self, source, where: str = "") -> int:
        specs = self.param_specs()
        check_names(specs, source.table(), where)
        fetch = Fetcher(source, self.opts.device, self.opts.dtype)
        self.load(fetch)
        return fetch.bytes_loaded

    def n_params(self) -> int:
        seen, n = set(), 0
        for s in self.param_specs():
            if s.absent or s.name in seen:
                continue
            seen.add(s.name)
            k = 1
            for d in s.shape:
                k *= d
            n += k
        return n

    def _reader_after(self, i: int, ctx):
        """The norm that reads the stream after run `i`, if what follows accepts rows prepared for it
        (`OwedNorm`) in this step: the next block's first norm, or the last norm before the head (only
        if every row's logits are wanted, in order)."""
        s = self.spec
        if i + 1 < len(s.schedule):
            first = getattr(s.layers[s.schedule[i + 1].layer], "first_norm", None)
            return first(ctx.n_tokens) if first is not None else None
        accepts = getattr(s.head, "accepts_owed_norm", None)
        if (ctx.wants_every_row and accepts is not None and accepts(ctx.n_tokens)
                and s.final_norm.deferred() is not None):
            return s.final_norm
        return None

    def forward(self, ctx, cache) -> torch.Tensor:
        """Runs the step described by `ctx`; returns float32 logits [n_want, vocab]."""
        s = self.spec
        stream = HiddenStream(s.embedding.forward(ctx.tokens, ctx.n_tokens))
        if s.position is not None:
            s.position.add_to_embeddings(stream.residual, ctx)
        for i, run in enumerate(s.schedule):
            view = self._views(i, cache, ctx.block_tables)
            stream.next_norm = self._reader_after(i, ctx)
            s.layers[run.layer].forward(stream, ctx, view, write_cache=run.reads_entry_of is None)
        stream.next_norm = None
        if ctx.n_want == 0:
            return torch.empty((0, s.vocab_size), dtype=torch.float32, device=stream.residual.device)
        if stream.owed is not None:
            if stream.owed.norm is not s.final_norm:
                raise RuntimeError("rows were prepared for another norm than the last one")
            h, stream.owed = stream.owed, None
        else:
            h = s.final_norm.forward(stream.residual, stream.delta, rows=ctx.want_rows, n_rows=ctx.n_want)
        return s.head.forward(h, n_rows=ctx.n_want)[:ctx.n_want]
