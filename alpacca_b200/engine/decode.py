"""Decode steps (one token per sequence) for the generation loop.

Two decoders with one interface, `step(live, more=None, stop=()) -> tokens`,
where `live` lists (slot, token to feed, sampler state) of the sequences still
running and the result is the next token of each.  `more[i]` says whether
sequence i has room for yet another step after this one, and `stop` holds the
tokens that end a sequence: with them a decoder knows, as soon as it has this
step's tokens, which sequences the caller will bring back, and may start their
next step before it returns (the caller must then come back with exactly those).

  EagerDecoder   one `Engine.step` and one sampler call per step; works for any model.
  GraphDecoder   the whole step - embedding to sampled token, and the feeding
                 back of that token - is captured once per batch shape in a CUDA
                 graph and replayed; the step's inputs live on the device and
                 advance there, so a step costs one graph launch and one small
                 read of the sampled tokens.  Rows of a batch shape that have no
                 sequence (padding up to the shape's size, or sequences that
                 ended) are marked and skipped by the kernels that touch the
                 cache; they change no result.

Both feed the same kernels in the same order, so they produce the same logits up
to the merge of attention chunks (the graph's chunk count is fixed by its shape).
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import PAGE_SIZE, CacheFull
from .step import StepContext, StepEntry, _pad4


class EagerDecoder:
    def __init__(self, engine, sampler):
        self.engine, self.sampler = engine, sampler

    def step(self, live, more=None, stop=()):
        logits = self.engine.step([StepEntry(slot, [tok], [0]) for slot, tok, _ in live])
        return self.sampler.sample(logits, [st for _, _, st in live])

    def run(self, live, steps: int):
        """`steps` steps, each token fed back; `live` is updated in place with the last tokens."""
        for _ in range(steps):
            tokens = self.step(live)
            live[:] = [(slot, t, st) for (slot, _, st), t in zip(live, tokens)]

    kernels_per_step = 0

    def close(self):
        pass


def bucket_rows(n: int) -> int:
    """Rows of the batch shape that holds n sequences."""
    for b in (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512, 768, 1024):
        if n <= b:
            return b
    return -(-n // 256) * 256


def _width_bucket(pages: int) -> int:
    """Block-table width (pages per sequence) of the batch shape that holds sequences of `pages` pages."""
    for b in (4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512, 768, 1024):
        if pages <= b:
            return b
    return -(-pages // 256) * 256


class _Shape:
    """Static device buffers and the captured graph of one batch shape (rows, block-table width)."""
    RING = 4        # more than the steps that are in flight at once

    def __init__(self, dec, rows: int, width: int):
        eng = dec.engine
        dev = eng.device
        self.rows, self.width = rows, width
        self.max_positions = eng.max_positions      # no sequence of this shape ever grows beyond it
        R = dec.window
        n_groups = len(eng.cache.kv_groups)
        names = ["tokens", "tok_seq", "tok_pos", "cu_q", "kv_len", "slots", "want_rows", "rng_stream", "rng_step",
                 "recent_pos", "seed", "row_order"]
        sizes = [rows, rows, rows, rows + 1, rows, rows, rows, rows, rows, rows, 2, rows]
        sizes += [rows * width] * n_groups + [rows * R]
        self.offs = [0]
        for s in sizes:
            self.offs.append(self.offs[-1] + _pad4(max(s, 1)))
        self.total = self.offs[-1]
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=dev)
        self.sect = {n: (self.offs[i], sizes[i]) for i, n in enumerate(names)}
        self.table_sect = [(self.offs[len(names) + g], rows * width) for g in range(n_groups)]
        self.recent_sect = (self.offs[len(names) + n_groups], rows * R)
        o, n = self.sect["tok_seq"]
        self.mask_host, self.mask_dev = self.host[o:o + n], self.dev[o:o + n]   # the live mask of the rows
        self.sampled = torch.zeros(rows, dtype=torch.int32, device=dev)
        # the tokens of the last steps, written by the step's last kernel itself into pinned host memory:
        # row (number of the replay) % RING; `replayed` counts the replays as the device's counter does
        self.host_ring = torch.zeros((self.RING, rows), dtype=torch.int32, pin_memory=True)
        self.replayed = 0
        self.history = torch.zeros((dec.history_len, rows), dtype=torch.int32, device=dev)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.graph = None
        self.logits = None      # set at capture: the logits of the last replay (after the repeat penalty)

    def d(self, name):
        o, n = self.sect[name]
        return self.dev[o:o + n]

    def h(self, name):
        o, n = self.sect[name]
        return self.host[o:o + n]

    def tables_dev(self):
        return [self.dev[o:o + n].view(self.rows, self.width) for o, n in self.table_sect]

    def tables_host(self):
        return [self.host[o:o + n].view(self.rows, self.width) for o, n in self.table_sect]

    def context(self) -> StepContext:
        return StepContext(
            n_tokens=self.rows, n_seqs=self.rows, n_want=self.rows, is_decode=True, max_q_len=1,
            max_kv_len=min(self.width * PAGE_SIZE, self.max_positions), tokens=self.d("tokens"), tok_seq=self.d("tok_seq"),
            tok_pos=self.d("tok_pos"), cu_q=self.d("cu_q"), kv_len=self.d("kv_len"), slots=self.d("slots"),
            want_rows=self.d("want_rows"), block_tables=self.tables_dev(), wants_every_row=True,
            row_order=self.d("row_order"))


class GraphDecoder:
    LOOKAHEAD = PAGE_SIZE      # pages are taken this many tokens ahead, so tables change rarely

    def __init__(self, engine, sampler, history_len: int = 512):
        if not engine.model.all_capturable():
            raise ValueError("this model has parts that cannot be captured in a CUDA graph")
        self.engine, self.sampler = engine, sampler
        p = sampler.params
        self.window = max(int(p.repeat_last_n), 1) if p.penalizes else 0
        self.history_len = int(history_len)
        self.shapes: dict[tuple, _Shape] = {}
        self.shape: _Shape | None = None
        self.layout: list = []          # slot of each row of the current shape
        self.row_of: dict = {}
        self.mask: list = []
        self.expect: dict = {}          # slot -> (length, last sampled token) after the last step
        self.pages_seen = -1
        self._last_slots, self._last_rows, self._room = None, None, 0
        self._flights: list = []        # steps that run ahead of the caller, oldest first

    # -- the captured step -------------------------------------------------------------
    def _body(self, sh: _Shape):
        eng, p = self.engine, self.sampler.params
        logits = eng.model.forward(sh.context(), eng.cache)
        sh.logits = logits      # float32 [rows, vocab] in the graph's own memory: every replay writes it anew
        o, n = sh.recent_sect
        recent = sh.dev[o:o + n].view(sh.rows, self.window) if self.window else None
        if recent is not None:
            ops.repeat_penalty(logits, recent, p.repeat_penalty)
        ops.sample(logits, sh.sampled, p.temperature, p.top_k, p.top_p if 0.0 < p.top_p < 1.0 else 1.0,
                   0, sh.d("rng_stream"), sh.d("rng_step"), seed_dev=sh.d("seed"))
        ops.decode_advance(sh.d("tokens"), sh.d("tok_pos"), sh.d("kv_len"), sh.d("rng_step"), sh.d("tok_seq"),
                           sh.sampled, recent, sh.d("recent_pos") if recent is not None else None, self.window,
                           sh.history, sh.counter, sh.rows, host_ring=sh.host_ring)

    def _capture(self, sh: _Shape):
        # with every row marked as padding the step touches neither cache nor counters, so the
        # warm-up run that must precede a capture is harmless
        sh.d("tok_seq").fill_(-1)
        sh.d("cu_q").copy_(torch.arange(sh.rows + 1, dtype=torch.int32))
        sh.d("want_rows").copy_(torch.arange(sh.rows, dtype=torch.int32))
        sh.d("row_order").copy_(torch.arange(sh.rows, dtype=torch.int32))
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._body(sh)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        sh.graph = torch.cuda.CUDAGraph()
        before = ops.launches
        with torch.cuda.graph(sh.graph):
            self._body(sh)
        sh.kernels = ops.launches - before      # kernels of this package in one replay
        sh.counter.zero_()
        sh.replayed = 0

    # -- layout ----------------------------------------------------------------------------
    def _reserve(self, live, steps: int):
        cache = self.engine.cache
        for slot, _, _ in live:
            left = cache.max_positions - cache.length(slot)
            if left < steps:
                raise CacheFull(f"context window full: slot {slot} holds {cache.length(slot)} tokens, "
                                f"{steps} more steps exceed the {cache.max_positions} positions of this engine")
        ahead = [(slot, min(max(steps, self.LOOKAHEAD), cache.max_positions - cache.length(slot)))
                 for slot, _, _ in live]
        try:
            cache.reserve(ahead)
        except CacheFull:
            cache.reserve([(slot, steps) for slot, _, _ in live])

    def _pages(self, live) -> int:
        g = self.engine.cache.kv_groups
        return sum(len(grp.page_lists[slot]) for grp in g for slot, _, _ in live)

    def _upload(self, live, tables_only: bool = False):
        sh, cache = self.shape, self.engine.cache
        slots = [slot for slot, _, _ in live] + [-1] * (sh.rows - len(live))
        for g, view in enumerate(sh.tables_host()):
            cache.fill_block_table(g, slots, view, sh.width)
        n = len(live)
        lens = [cache.length(slot) for slot, _, _ in live]
        sh.h("tokens").zero_()
        sh.h("tokens")[:n] = torch.tensor([tok for _, tok, _ in live], dtype=torch.int32)
        sh.h("tok_seq").fill_(-1)
        sh.h("tok_seq")[:n] = torch.arange(n, dtype=torch.int32)
        sh.h("tok_pos").zero_()
        sh.h("tok_pos")[:n] = torch.tensor(lens, dtype=torch.int32)
        sh.h("cu_q").copy_(torch.arange(sh.rows + 1, dtype=torch.int32))
        sh.h("kv_len").zero_()
        sh.h("kv_len")[:n] = torch.tensor(lens, dtype=torch.int32) + 1
        sh.h("slots").copy_(torch.tensor(slots, dtype=torch.int32))
        # the rows, longest sequence first (the sequences grow in step, so the order holds for the
        # layout's life); rows without a sequence come last
        sh.h("row_order").copy_(torch.tensor(sorted(range(sh.rows), key=lambda r: -lens[r] if r < n else 1),
                                             dtype=torch.int32))
        sh.h("want_rows").copy_(torch.arange(sh.rows, dtype=torch.int32))
        sh.h("rng_stream").zero_()
        sh.h("rng_stream")[:n] = torch.tensor([st.stream for _, _, st in live], dtype=torch.int32)
        sh.h("rng_step").zero_()
        sh.h("rng_step")[:n] = torch.tensor([st.step for _, _, st in live], dtype=torch.int32)
        seed = self.sampler.seed & (2 ** 64 - 1)
        sh.h("seed").copy_(torch.tensor([seed & 0xFFFFFFFF, seed >> 32], dtype=torch.int64).to(torch.int32))
        if self.window:
            o, m = sh.recent_sect
            rec = sh.host[o:o + m].view(sh.rows, self.window)
            rec.fill_(-1)
            sh.h("recent_pos").zero_()
            for b, (_, _, st) in enumerate(live):
                r = st.recent[-self.window:]
                rec[b, :len(r)] = torch.tensor(r, dtype=torch.int32)
                sh.h("recent_pos")[b] = len(r) % self.window
        sh.dev.copy_(sh.host, non_blocking=True)

    def _prepare(self, live, steps: int, always_mask: bool = False):
        """Makes the device state fit `live`.  Rows keep their sequence for the life of a layout;
        a sequence that ended is masked out (its row becomes padding) until so few are left that a
        smaller shape pays.  Returns the row of each live sequence."""
        cache = self.engine.cache
        slots = [slot for slot, _, _ in live]
        sh = self.shape
        # the usual case, kept short: the same sequences as in the last step, each continued exactly
        # where that step left it, with room left in the pages they hold
        if (sh is not None and slots == self._last_slots and self._room >= steps
                and all(self.expect.get(slot) in ((cache.length(slot), tok), (cache.length(slot), None))
                        for slot, tok, _ in live)):
            self._room -= steps
            if always_mask:
                sh.mask_dev.copy_(sh.mask_host, non_blocking=True)
            return self._last_rows
        rows = self._prepare_slow(live, steps, always_mask)
        self._last_slots, self._last_rows = slots, rows
        # steps that need nothing from the host: room in the pages held and in the context
        self._room = min([len(g.page_lists[s]) * PAGE_SIZE - cache.length(s) for g in cache.kv_groups for s in slots]
                         + [cache.max_positions - cache.length(s) for s in slots]) - steps
        return rows

    def _prepare_slow(self, live, steps: int, always_mask: bool):
        cache = self.engine.cache
        self._reserve(live, steps)
        need_pages = max([len(grp.page_lists[slot]) for grp in cache.kv_groups for slot, _, _ in live] + [1])
        slots = [slot for slot, _, _ in live]
        sh = self.shape
        # the device state is only valid for sequences that went on exactly as the last step left them
        fresh = all(self.expect.get(slot) in ((cache.length(slot), tok), (cache.length(slot), None))
                    for slot, tok, _ in live)
        keep = (sh is not None and fresh and all(s in self.row_of for s in slots) and sh.width >= need_pages
                and bucket_rows(len(slots)) * 2 > sh.rows)
        if not keep:
            key = (bucket_rows(len(live)), _width_bucket(need_pages))
            sh = self.shapes.get(key)
            if sh is None:
                sh = _Shape(self, *key)
                self._capture(sh)
                self.shapes[key] = sh
            torch.cuda.current_stream().synchronize()      # the pinned staging buffer is free again
            self.shape, self.layout = sh, slots
            self.row_of = {s: r for r, s in enumerate(slots)}
            self._upload(live, tables_only=False)
            self.pages_seen = self._pages(live)
            self.mask = list(range(len(slots))) + [-1] * (sh.rows - len(slots))
            return list(range(len(slots)))
        rows = [self.row_of[s] for s in slots]
        if self._pages(live) != self.pages_seen:
            torch.cuda.current_stream().synchronize()
            full = [(self.layout[r], None, None) for r in range(len(self.layout))]
            self._upload_tables(full)
            self.pages_seen = self._pages(live)
        alive = set(rows)
        mask = [r if r in alive else -1 for r in range(sh.rows)]
        if mask != self.mask or always_mask:
            if mask != self.mask:
                torch.cuda.current_stream().synchronize()
            self.mask = mask
            sh.mask_host.copy_(torch.tensor(mask, dtype=torch.int32))
            sh.mask_dev.copy_(sh.mask_host, non_blocking=True)
        return rows

    def _upload_tables(self, layout_entries):
        sh, cache = self.shape, self.engine.cache
        slots = [s if cache.slots.is_held(s) and s in cache.lengths else -1 for s, _, _ in layout_entries]
        slots += [-1] * (sh.rows - len(slots))
        for g, view in enumerate(sh.tables_host()):
            cache.fill_block_table(g, slots, view, sh.width)
        for o, n in sh.table_sect:
            sh.dev[o:o + n].copy_(sh.host[o:o + n], non_blocking=True)

    # -- stepping ------------------------------------------------------------------------------
    @property
    def kernels_per_step(self) -> int:
        return self.shape.kernels if self.shape is not None else 0

    def run(self, live, steps: int, always_mask: bool = False):
        """`steps` decode steps on the device without reading anything back.  The host's view of
        lengths is advanced; the sampled tokens stay in the shape's history ring."""
        rows = self._prepare(live, steps, always_mask)
        for _ in range(steps):
            self.shape.graph.replay()
        self.shape.replayed += steps
        cache = self.engine.cache
        cache.commit([(slot, steps) for slot, _, _ in live])
        self.expect = {slot: (cache.length(slot), None) for slot, _, _ in live}
        return rows

    def _launch(self, live):
        """Enqueues one step for `live`; its tokens arrive in a row of the shape's pinned ring (written by the
        step's last kernel), to be read once the event recorded behind the step has passed."""
        rows = self.run(live, 1, always_mask=True)
        sh = self.shape
        host = sh.host_ring[(sh.replayed - 1) % sh.RING]      # where this replay's last kernel writes its tokens
        done = torch.cuda.Event()
        done.record()
        return {"live": list(live), "rows": rows, "done": done, "host": host}

    def _drop_flights(self, live):
        """Gives up the steps that ran ahead for sequences the caller did not bring back: their tokens
        are dropped, the lengths they were counted with are taken back, the device state is uploaded
        anew by the next step."""
        flights, self._flights = self._flights, []
        flights[-1]["done"].synchronize()
        # a sequence is known by its sampler state: one that the caller still brings has the steps
        # that ran ahead in its length; one that is gone has given its slot back
        here = {id(st) for _, _, st in live}
        for f in flights:
            self.engine.cache.commit([(slot, -1) for slot, _, st in f["live"] if id(st) in here])
        sampler = self.sampler
        self.reset()
        self.sampler = sampler

    def settle(self, live) -> None:
        """Gives up the steps that run ahead, if there are any (`live`: the sequences still running,
        as they would be brought to the next step), so that lengths are what the caller has seen."""
        if self._flights:
            self._drop_flights(live)

    def step(self, live, more=None, stop=()):
        """One step: the live mask goes to the device (a small copy from pinned memory), the graph
        is replayed, the sampled tokens come back.

        With `more`, up to two further steps are enqueued before this step's tokens are returned, so
        that the device never waits for the host: the next step of all sequences that have room for
        one is enqueued before this step's tokens are even known (it feeds on the tokens on the
        device), provided that needs nothing from the host but the replay.  If one of them then
        samples a stop token, the caller comes back without it, and the step that ran ahead is given
        up: one step's worth of device time for each sequence end by a stop token."""
        q = self._flights
        if q and [(slot, tok) for slot, tok, _ in q[0]["live"]] != [(slot, tok) for slot, tok, _ in live]:
            self._drop_flights(live)
            q = self._flights
        if not q:
            q.append(self._launch(live))
        slots = [slot for slot, _, _ in live]
        if more is not None and len(q) == 1 and all(more) and slots == self._last_slots and self._room >= 1:
            q.append(self._launch([(slot, None, st) for slot, _, st in live]))
        flight = q.pop(0)
        flight["done"].synchronize()
        got = flight["host"].tolist()
        tokens = [got[r] for r in flight["rows"]]
        for (slot, _, st), t in zip(live, tokens):
            st.step += 1
            st.accept(t)
            if not q:
                self.expect[slot] = (self.expect[slot][0], t)
        if q:
            # the step that ran ahead fed on these tokens
            q[0]["live"] = [(slot, t, st) for (slot, _, st), t in zip(live, tokens)]
        elif more is not None:
            ahead = [(slot, t, st) for (slot, _, st), t, m in zip(live, tokens, more) if m and t not in stop]
            if ahead:
                q.append(self._launch(ahead))
        return tokens

    def history(self, n_steps: int, n_live: int) -> torch.Tensor:
        """The sampled tokens of the last `n_steps` steps of the current shape, [n_steps, n_live] (host)."""
        sh = self.shape
        count = int(sh.counter.item())
        idx = [(count - n_steps + i) % self.history_len for i in range(n_steps)]
        return sh.history[idx][:, :n_live].cpu()

    def reset(self, sampler=None) -> None:
        """Forgets the device layout (the next step uploads everything anew); optionally takes
        another sampler with the same options but its own seed."""
        if sampler is not None:
            self.sampler = sampler
        if self._flights:
            self._flights[-1]["done"].synchronize()
            self._flights = []
        self.shape, self.layout, self.row_of, self.mask, self.pages_seen = None, [], {}, [], -1
        self.expect = {}
        self._last_slots, self._last_rows, self._room = None, None, 0

    def close(self):
        self.shapes.clear()
        self.shape = None
