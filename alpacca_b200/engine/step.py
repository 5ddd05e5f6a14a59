"""One step's batch, as the kernels see it.

A step runs a batch of sequences, each with one or more new tokens on top of
what its slot already holds.  The tokens are packed one sequence after another
(no padding between them); every per-token and per-sequence index lives in one
int32 buffer that is copied to the device once per step.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepEntry:
    slot: int
    tokens: list            # the sequence's next tokens (at least one)
    want: list = field(default_factory=list)   # indices into `tokens` whose logits are wanted


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    n_want: int
    is_decode: bool          # every sequence brings exactly one token
    max_q_len: int
    max_kv_len: int
    tokens: torch.Tensor     # int32 [n_tokens]   token ids, packed
    tok_seq: torch.Tensor    # int32 [n_tokens]   batch row of each token (-1: padding)
    tok_pos: torch.Tensor    # int32 [n_tokens]   position of each token in its sequence
    cu_q: torch.Tensor       # int32 [n_seqs+1]   start of each sequence's tokens in the packing
    kv_len: torch.Tensor     # int32 [n_seqs]     sequence length after this step
    slots: torch.Tensor      # int32 [n_seqs]     slot of each batch row (-1: padding)
    want_rows: torch.Tensor  # int32 [n_want]     packed rows whose logits are wanted
    block_tables: list       # per key/value group: int32 [n_seqs, W]
    host_slots: list = None      # the same facts on the host, for parts that plan on the host
    host_q_lens: list = None
    host_kv_lens: list = None
    wants_every_row: bool = False    # want_rows is 0, 1, .., n_tokens - 1: each row's logits, in order
    row_order: torch.Tensor = None   # int32 [n_seqs], decode steps: the batch rows, longest sequence first
                                     # (kernels that give a row to a CTA start the long rows first)
    extras: dict = field(default_factory=dict)   # per-step plans of kernels (tile lists and the like)
    buffer: torch.Tensor = None      # the one device buffer that all the index arrays above are views of


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class ContextBuilder:
    """Packs the step's index arrays into a pinned staging buffer and copies them over."""

    RING = 4

    def __init__(self, device):
        self.device = torch.device(device)
        self.pinned = self.device.type == "cuda"
        self._ring = [None] * self.RING
        self._events = [None] * self.RING
        self._turn = 0

    def _staging(self, n: int) -> torch.Tensor:
        i = self._turn
        self._turn = (self._turn + 1) % self.RING
        if self._events[i] is not None:
            self._events[i].synchronize()     # the copy that last used this buffer is done
        buf = self._ring[i]
        if buf is None or buf.numel() < n:
            cap = max(4096, 1 << (n - 1).bit_length())
            buf = torch.empty(cap, dtype=torch.int32, pin_memory=self.pinned)
            self._ring[i] = buf
        self._slot = i
        return buf

    def build(self, entries, lengths, cache, token_arrays=None, into: torch.Tensor | None = None,
              widths=None) -> StepContext:
        """`into`: the `buffer` of a context built earlier for a step of the same shape (the same numbers of
        tokens, sequences, wanted places and pages): the arrays are written there instead of into new memory,
        and nothing is returned (that context's views see them).  `widths`: the block tables' widths, one per
        key/value group, if they are to be wider than the longest sequence needs (the rest is zero)."""
        B = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        n_want = sum(len(e.want) for e in entries)
        if widths is None:
            widths = [cache.table_width(g, [e.slot for e in entries]) for g in range(len(cache.kv_groups))]
        decode = all(q == 1 for q in q_lens)
        sizes = [T, T, T, B + 1, B, B, n_want] + [B * w for w in widths] + [B if decode else 0]
        offs = [0]
        for s in sizes:
            offs.append(offs[-1] + _pad4(max(s, 1)))
        total = offs[-1]
        stage = self._staging(total)
        host = stage.numpy()
        if token_arrays is None:
            token_arrays = [np.asarray(e.tokens, dtype=np.int32) for e in entries]
        host[offs[0]:offs[0] + T] = token_arrays[0] if B == 1 else np.concatenate(token_arrays)
        cu = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu[1:])
        host[offs[1]:offs[1] + T] = np.repeat(np.arange(B, dtype=np.int32), q_lens)
        starts = np.repeat(np.asarray(lengths, dtype=np.int32) - cu[:-1], q_lens)
        host[offs[2]:offs[2] + T] = starts + np.arange(T, dtype=np.int32)
        host[offs[3]:offs[3] + B + 1] = cu
        kv = np.asarray(lengths, dtype=np.int32) + np.asarray(q_lens, dtype=np.int32)
        host[offs[4]:offs[4] + B] = kv
        host[offs[5]:offs[5] + B] = [e.slot for e in entries]
        if n_want:
            host[offs[6]:offs[6] + n_want] = [int(cu[b]) + w for b, e in enumerate(entries) for w in e.want]
        for g, w in enumerate(widths):
            view = stage[offs[7 + g]:offs[7 + g] + B * w].view(B, w)
            cache.fill_block_table(g, [e.slot for e in entries], view, w)
        i_order = 7 + len(widths)
        if decode:
            host[offs[i_order]:offs[i_order] + B] = np.argsort(-kv, kind="stable")
        if into is not None:
            if into.numel() != total:
                raise ValueError(f"a step of another shape than the buffer's ({total} against {into.numel()} entries)")
            dev = into
        else:
            dev = torch.empty(total, dtype=torch.int32, device=self.device)
        dev.copy_(stage[:total], non_blocking=True)
        if self.pinned:
            ev = torch.cuda.Event()
            ev.record()
            self._events[self._slot] = ev
        if into is not None:
            return None         # the context that owns `into` has its views already

        def part(i, n):
            return dev[offs[i]:offs[i] + n]
        return StepContext(
            buffer=dev, n_tokens=T, n_seqs=B, n_want=n_want, is_decode=decode, row_order=part(i_order, B) if decode else None,
            max_q_len=max(q_lens), max_kv_len=int(kv.max()),
            tokens=part(0, T), tok_seq=part(1, T), tok_pos=part(2, T), cu_q=part(3, B + 1),
            kv_len=part(4, B), slots=part(5, B), want_rows=part(6, n_want),
            block_tables=[dev[offs[7 + g]:offs[7 + g] + B * w].view(B, w) for g, w in enumerate(widths)],
            host_slots=[e.slot for e in entries], host_q_lens=q_lens, host_kv_lens=kv.tolist(),
            wants_every_row=all(len(e.want) == q and all(w == i for i, w in enumerate(e.want))
                                for e, q in zip(entries, q_lens)))
