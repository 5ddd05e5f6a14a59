"""The cache of the sequences in flight.

A *slot* stands for one sequence of a batch: its length, its pages in every
key/value group and its row in every state group.  Storage is per *group* of
cache entries with the same needs:

  KVGroup     keys and values [entry, page, kv_head, position-in-page, head_dim],
              in pages of PAGE_SIZE positions that sequences take as they grow
              and give back when they end; a group with a window gives pages
              back as soon as they lie wholly before the window;
  StateGroup  a state of fixed shape per (entry, slot), zeroed when the slot
              is taken.

An *entry* is one run of a layer in the model's schedule that owns cache of its
own (a run that reads another run's cache has none).  The reference keeps one
sequence only: per layer two arrays [n_ctx, n_kv, head_dim] and the counter
`n_past` (alpacca/model.py:345-362); `reset()` there is `free_slot` here.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import KVSpec, StateSpec
from .pool import CacheFull, IdPool

PAGE_SIZE = 64


@dataclass
class KVLayerView:
    """What an attention mixer gets: its entry's pages and the step's block table."""
    k: torch.Tensor            # [n_pages, K, PAGE_SIZE, D]
    v: torch.Tensor
    block_table: torch.Tensor  # int32 [B, W]: page of position p of batch row b at [b, p // PAGE_SIZE]
    group: "KVGroup"


@dataclass
class StateLayerView:
    """What a mixer with state gets: state[slot] is its sequence's state."""
    state: torch.Tensor        # [max_slots, *shape]
    group: "StateGroup"


class KVGroup:
    def __init__(self, spec: KVSpec, n_entries: int, n_pages: int, dtype, device):
        self.spec, self.n_entries, self.n_pages = spec, n_entries, int(n_pages)
        shape = (n_entries, self.n_pages, spec.n_kv_heads, PAGE_SIZE, spec.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pages = IdPool(self.n_pages, "cache page")
        self.page_lists: dict[int, list[int]] = {}   # slot -> page of each page index (-1: given back)

    @property
    def bytes_per_token(self) -> int:
        return 2 * self.n_entries * self.spec.n_kv_heads * self.spec.head_dim * self.k.element_size()

    def open(self, slot: int) -> None:
        self.page_lists[slot] = []

    def pages_needed(self, slot: int, new_len: int) -> int:
        return max(0, -(-new_len // PAGE_SIZE) - len(self.page_lists[slot]))

    def grow(self, slot: int, new_len: int) -> None:
        pl = self.page_lists[slot]
        pl.extend(self.pages.alloc_many(self.pages_needed(slot, new_len)))

    def release_before(self, slot: int, first_needed_pos: int) -> None:
        """Gives back pages that hold only positions before `first_needed_pos` (window groups)."""
        pl = self.page_lists[slot]
        for i in range(min(first_needed_pos // PAGE_SIZE, len(pl))):
            if pl[i] >= 0:
                self.pages.free(pl[i])
                pl[i] = -1

    def holds_from(self, slot: int, first_pos: int, new_len: int) -> bool:
        """Whether the pages of positions first_pos .. new_len - 1 are still held (a window gives pages back)."""
        pl = self.page_lists[slot]
        return all(pl[i] >= 0 for i in range(first_pos // PAGE_SIZE, min(-(-new_len // PAGE_SIZE), len(pl))))

    def shrink(self, slot: int, new_len: int) -> None:
        """Gives back the pages that hold only positions from `new_len` on."""
        pl = self.page_lists[slot]
        for p in pl[-(-new_len // PAGE_SIZE):]:
            if p >= 0:
                self.pages.free(p)
        del pl[-(-new_len // PAGE_SIZE):]

    def close(self, slot: int) -> None:
        for p in self.page_lists.pop(slot):
            if p >= 0:
                self.pages.free(p)

    def live_tokens(self, lengths: dict[int, int]) -> int:
        return sum(sum(1 for p in pl if p >= 0) for pl in self.page_lists.values()) * PAGE_SIZE


class StateGroup:
    def __init__(self, spec: StateSpec, n_entries: int, max_slots: int, device):
        self.spec, self.n_entries = spec, n_entries
        self.state = torch.zeros((n_entries, max_slots, *spec.shape), dtype=spec.dtype, device=device)

    def open(self, slot: int) -> None:
        self.state[:, slot].zero_()


class SequenceCache:
    """Slots, their lengths, and the groups of storage behind them.

    `entry_specs`: for each cache entry of the schedule its `KVSpec`,
    `StateSpec` or None.  Entries with equal specs share a group.
    """

    def __init__(self, entry_specs, max_tokens: int, max_slots: int, max_positions: int, dtype, device):
        self.device = device
        self.max_positions = int(max_positions)
        self.n_pages = max(1, -(-int(max_tokens) // PAGE_SIZE))
        self.slots = IdPool(int(max_slots), "slot")
        self.lengths: dict[int, int] = {}
        self.kv_groups: list[KVGroup] = []
        self.state_groups: list[StateGroup] = []
        self.entry_place: list[tuple[str, int, int] | None] = []   # (kind, group, index within group)
        by_spec: dict = {}
        for spec in entry_specs:
            if spec is None:
                self.entry_place.append(None)
                continue
            by_spec.setdefault(spec, []).append(len(self.entry_place))
            self.entry_place.append(("pending", 0, 0))
        for spec, entries in by_spec.items():
            if isinstance(spec, KVSpec):
                g = len(self.kv_groups)
                self.kv_groups.append(KVGroup(spec, len(entries), self.n_pages, dtype, device))
                kind = "kv"
            elif isinstance(spec, StateSpec):
                g = len(self.state_groups)
                self.state_groups.append(StateGroup(spec, len(entries), int(max_slots), device))
                kind = "state"
            else:
                raise TypeError(f"cache spec {spec!r} is neither KVSpec nor StateSpec")
            for j, e in enumerate(entries):
                self.entry_place[e] = (kind, g, j)

    # -- slots ---------------------------------------------------------------
    def alloc_slot(self) -> int:
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        for g in self.kv_groups:
            g.open(slot)
        for g in self.state_groups:
            g.open(slot)
        return slot

    def free_slot(self, slot: int) -> None:
        if slot not in self.lengths:
            raise ValueError(f"slot {slot} is freed twice (or was never given out)")
        for g in self.kv_groups:
            g.close(slot)
        del self.lengths[slot]
        self.slots.free(slot)

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    # -- growth ----------------------------------------------------------------
    def reserve(self, requests) -> None:
        """Makes room for `n_new` more tokens in each (slot, n_new) of `requests`, or raises
        CacheFull and changes nothing."""
        for slot, n_new in requests:
            if slot not in self.lengths:
                raise ValueError(f"slot {slot} is not in use")
            if self.lengths[slot] + n_new > self.max_positions:
                raise CacheFull(f"context window full: slot {slot} holds {self.lengths[slot]} tokens, "
                                f"{n_new} more exceed the {self.max_positions} positions of this engine")
        for g in self.kv_groups:
            if g.spec.window:
                for slot, _ in requests:
                    g.release_before(slot, self.lengths[slot] - g.spec.window + 1)
            need = sum(g.pages_needed(slot, self.lengths[slot] + n_new) for slot, n_new in requests)
            if need > g.pages.n_free:
                raise CacheFull(f"cache full: {need} more pages of {PAGE_SIZE} tokens wanted, "
                                f"{g.pages.n_free} of {g.n_pages} free")
        for g in self.kv_groups:
            for slot, n_new in requests:
                g.grow(slot, self.lengths[slot] + n_new)

    def commit(self, requests) -> None:
        for slot, n_new in requests:
            self.lengths[slot] += n_new

    def truncate(self, slot: int, n: int) -> None:
        """Keeps only the first `n` tokens of `slot` (the reference's `_truncate_cache`,
        alpacca/model.py:367-377): the length is set back and the pages that lie wholly behind it
        are given back; what a kept page holds after position n - 1 is never read.  Refused, with
        nothing changed, where it cannot be undone: a state of fixed size has no earlier value, and
        a group with a window may have given back pages that the shorter sequence would read."""
        if slot not in self.lengths:
            raise ValueError(f"slot {slot} is not in use")
        cur = self.lengths[slot]
        if not 0 <= n <= cur:
            raise ValueError(f"slot {slot} holds {cur} tokens; it cannot be truncated to {n}")
        if n == cur:
            return
        if self.state_groups:
            raise ValueError("a sequence whose model keeps a state of fixed size cannot be truncated "
                             "(the state has no earlier value); free the slot and start again")
        for g in self.kv_groups:
            if g.spec.window and not g.holds_from(slot, max(0, n - g.spec.window + 1), n):
                raise ValueError(f"slot {slot}: pages before position {n} that the window of "
                                 f"{g.spec.window} needs were already given back")
        for g in self.kv_groups:
            g.shrink(slot, n)
        self.lengths[slot] = n

    # -- views -----------------------------------------------------------------
    def table_width(self, group: int, slots) -> int:
        g = self.kv_groups[group]
        return max([len(g.page_lists[s]) for s in slots if s >= 0] + [1])

    def fill_block_table(self, group: int, slots, out, width: int) -> None:
        """Writes the page lists of `slots` into `out` (a host int32 tensor [len(slots), width])."""
        g = self.kv_groups[group]
        table = out.numpy()         # the same memory; filling it row by row through torch costs 10 us a row
        table[:] = 0
        for b, s in enumerate(slots):
            if s < 0:
                continue
            pl = g.page_lists[s]
            if pl:
                table[b, :len(pl)] = pl
                if g.spec.window:           # pages that a window has given back are marked -1 in the list
                    table[b, :len(pl)].clip(0, None, out=table[b, :len(pl)])

    def entry_view(self, entry: int, block_tables) -> KVLayerView | StateLayerView | None:
        place = self.entry_place[entry]
        if place is None:
            return None
        kind, g, j = place
        if kind == "kv":
            grp = self.kv_groups[g]
            return KVLayerView(grp.k[j], grp.v[j], block_tables[g], grp)
        grp = self.state_groups[g]
        return StateLayerView(grp.state[j], grp)

    # -- accounting ----------------------------------------------------------------
    def check(self) -> None:
        """Raises if a page or slot is lost, held twice, or held by nobody."""
        self.slots.check()
        assert set(self.lengths) == {i for i in range(self.slots.n) if self.slots.is_held(i)}
        for g in self.kv_groups:
            g.pages.check()
            held = [p for pl in g.page_lists.values() for p in pl if p >= 0]
            assert len(held) == len(set(held)), "a cache page belongs to two sequences"
            assert len(held) == g.pages.n_held, "cache pages are held that no sequence owns"
            assert set(g.page_lists) == set(self.lengths)

    def describe(self) -> str:
        kv = sum(g.k.numel() * g.k.element_size() * 2 for g in self.kv_groups)
        st = sum(g.state.numel() * g.state.element_size() for g in self.state_groups)
        return (f"cache: {self.n_pages} pages of {PAGE_SIZE} tokens in {len(self.kv_groups)} key/value group(s) "
                f"({kv / 2**20:.1f} MiB), {len(self.state_groups)} state group(s) ({st / 2**20:.1f} MiB), "
                f"{self.slots.n} slots")
