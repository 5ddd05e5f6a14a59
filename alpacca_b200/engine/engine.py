"""The engine: a model, its cache, and the one step function.

`Engine.step(entries)` runs exactly the tokens it is given, on top of what the
slots hold, as one batch, and returns the logits at the wanted places.  Prompts
of unequal lengths go in one step; afterwards one token per sequence.  The
reference's counterparts are `prefill` / `forward_batch` / `forward`
(alpacca/model.py:610-641, :469-518, :439-445), for its single sequence.

A step whose shape was seen before is replayed from a CUDA graph: the second step of a shape is run
launch by launch on index arrays that stay where they are and is captured afterwards, later ones copy
their token ids, slots, pages and wanted places into those arrays and replay.  The shape of a prompt step
is the numbers of new and held tokens of every sequence and of wanted places per sequence; of a step of
one token each, the number of sequences and the width of the block tables (lengths are data there).  A
step of 2,048 tokens of the 1B shape takes 3.8 ms of device time and 4.4 ms when the host issues its 130
launches one by one; a step of one token 0.65 ms against about 2 ms.
"""
from __future__ import annotations

from collections import OrderedDict

import numpy as np
import torch

from .. import ops
from ..cache import CacheFull, SequenceCache
from ..parts.base import BuildOptions
from .model import DecoderModel
from .step import ContextBuilder, StepContext, StepEntry


class Engine:
    def __init__(self, model: DecoderModel, max_tokens: int, max_slots: int | None = None,
                 max_positions: int | None = None):
        self.model = model
        opts: BuildOptions = model.opts
        self.device = torch.device(opts.device)
        self.max_positions = int(max_positions or opts.max_positions)
        if not 0 < self.max_positions <= opts.max_positions:
            # tables indexed by position (the rotation's angles) have opts.max_positions rows
            raise ValueError(f"an engine of {self.max_positions} positions was asked for, the model was built "
                             f"for {opts.max_positions}")
        n_pages = -(-int(max_tokens) // 64)
        self.max_slots = int(max_slots) if max_slots else max(1, min(n_pages, 1024))
        self.cache = SequenceCache(model.cache_entry_specs(), max_tokens, self.max_slots, self.max_positions,
                                   opts.dtype, self.device)
        self.vocab_size = model.spec.vocab_size
        self._builder = ContextBuilder(self.device)
        # steps replayed from graphs: shape -> times seen, shape -> (context, graph, logits)
        self.step_graphs = self.device.type == "cuda" and model.all_capturable()
        self._shapes_seen: dict = {}
        self._graphs: OrderedDict = OrderedDict()

    # -- slots -------------------------------------------------------------
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def truncate(self, slot: int, n: int) -> None:
        """Keeps only the first `n` tokens of the slot's sequence (see `SequenceCache.truncate`)."""
        self.wait()          # steps in flight still read what is given back
        self.cache.truncate(slot, n)

    def wait(self) -> None:
        """Returns when every step issued so far has run (steps are issued asynchronously), and
        raises if a kernel of theirs reported that it gave up (see `ops.check_tc_status`)."""
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
            ops.check_tc_status()

    def room_for(self, token_counts) -> bool:
        """Whether new sequences of these lengths fit together into what is free now."""
        pages = sum(-(-int(n) // 64) for n in token_counts)
        return (len(token_counts) <= self.cache.slots.n_free
                and all(pages <= g.pages.n_free for g in self.cache.kv_groups))

    # -- the step ------------------------------------------------------------
    def _check(self, entries) -> list:
        """Refuses a step that the kernels must not see; returns each entry's tokens as an int32 array."""
        if not entries:
            raise ValueError("a step needs at least one sequence")
        seen = set()
        arrays = []
        for e in entries:
            if e.slot in seen:
                raise ValueError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if len(e.tokens) == 0:
                raise ValueError(f"slot {e.slot}: a step needs at least one token per sequence")
            ids = np.asarray(e.tokens)
            if ids.ndim != 1 or ids.dtype.kind not in "iu":
                raise ValueError(f"slot {e.slot}: token ids must be a flat list of integers")
            lo, hi = int(ids.min()), int(ids.max())
            if lo < 0 or hi >= self.vocab_size:
                bad = lo if lo < 0 else hi
                raise ValueError(f"token id {bad} lies outside the vocabulary of {self.vocab_size}")
            arrays.append(ids.astype(np.int32, copy=False))
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"slot {e.slot}: wanted place {w} is not among its {len(e.tokens)} tokens")
        return arrays

    def prepare(self, entries) -> StepContext:
        arrays = self._check(entries)
        requests = [(e.slot, len(e.tokens)) for e in entries]
        self.cache.reserve(requests)          # raises CacheFull before anything is launched
        lengths = [self.cache.length(e.slot) for e in entries]
        return self._builder.build(entries, lengths, self.cache, arrays)

    PROMPT_GRAPH_MAX_TOKENS = 8192      # longer steps are bound by the device, not by the host that issues them
    STEP_GRAPHS_KEPT = 16

    def _shape_of(self, entries, lengths):
        """(shape, block-table widths): what decides every launch of a step (the rest - token ids, slots,
        pages, wanted places, and for single-token steps the lengths too - is data in device memory); the
        shape is None for steps that are not replayed from graphs."""
        q_lens = tuple(len(e.tokens) for e in entries)
        slots = [e.slot for e in entries]
        widths = tuple(self.cache.table_width(g, slots) for g in range(len(self.cache.kv_groups)))
        if not self.step_graphs or sum(q_lens) > self.PROMPT_GRAPH_MAX_TOKENS or ops.timing():
            return None, widths
        wants = tuple(len(e.want) for e in entries)
        every = all(len(e.want) == q and all(w == i for i, w in enumerate(e.want)) for e, q in zip(entries, q_lens))
        if max(q_lens) == 1:
            # one token each: the kernels take the lengths from device memory; tables as wide as the batch
            # shapes of the graph decoder are, so that a shape lasts for many steps
            from .decode import _width_bucket
            widths = tuple(_width_bucket(w) for w in widths)
            return ("one token each", len(entries), wants, every, widths), widths
        return (q_lens, tuple(lengths), wants, every, widths), widths

    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        """Runs one step; returns float32 logits [number of wanted places, vocab] on the device,
        in the order of the entries and of their `want` lists."""
        arrays = self._check(entries)
        requests = [(e.slot, len(e.tokens)) for e in entries]
        self.cache.reserve(requests)          # raises CacheFull before anything is launched
        lengths = [self.cache.length(e.slot) for e in entries]
        shape, widths = self._shape_of(entries, lengths)
        held = self._graphs.get(shape) if shape is not None else None
        capture = None
        if held is not None:
            ctx, graph, logits = held
            self._graphs.move_to_end(shape)
            self._builder.build(entries, lengths, self.cache, arrays, into=ctx.buffer, widths=widths)
            graph.replay()
            logits = logits.clone()           # the graph's own memory is written again by its next replay
        else:
            ctx = self._builder.build(entries, lengths, self.cache, arrays, widths=widths)
            logits = self.model.forward(ctx, self.cache)
            if shape is not None:
                seen = self._shapes_seen[shape] = self._shapes_seen.get(shape, 0) + 1
                if seen == 2:
                    capture = ctx
        self.cache.commit(requests)
        if capture is not None:
            self._capture(shape, capture)
        return logits

    def _capture(self, shape, ctx) -> None:
        """Captures the step that was just issued with `ctx` (whose plans, made on the host during that run,
        stay with it) for later steps of the same shape.  Nothing runs during the capture."""
        graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx, self.cache)
        except Exception as e:       # noqa: BLE001 - the step itself has run and is committed; only the replay is lost
            import warnings
            warnings.warn(f"a step could not be captured in a CUDA graph ({e}); steps are issued launch by "
                          "launch from now on", RuntimeWarning, stacklevel=3)
            self.step_graphs = False
            self._graphs.clear()
            return
        self._graphs[shape] = (ctx, graph, logits)
        while len(self._graphs) > self.STEP_GRAPHS_KEPT:
            self._graphs.popitem(last=False)
        if len(self._shapes_seen) > 4096:
            self._shapes_seen.clear()

    def forget_graphs(self) -> None:
        """Drops the captured steps: the next steps of every shape are issued launch by launch again (for a
        caller that has changed what a step launches, such as a switch of `ops`)."""
        self._graphs.clear()
        self._shapes_seen.clear()

    def describe(self) -> str:
        return self.cache.describe()


__all__ = ["Engine", "StepEntry", "CacheFull"]
