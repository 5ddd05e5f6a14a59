"""The block's decisions about the norm that runs inside the products around it (`OwedNorm`),
with stand-in parts on the CPU: who is offered `then`, who is handed prepared rows, and that
parts which define none of it are run exactly as without it."""
import pytest
import torch

from alpacca_b200.parts.base import FeedForward, Mixer, Norm, OwedNorm
from alpacca_b200.parts.block import HiddenStream, PreNormBlock


class Ctx:
    n_tokens = 3


class PlainNorm(Norm):
    """A norm that cannot be deferred: adds the delta, returns the residual."""

    def __init__(self):
        self.calls = 0

    def forward(self, residual, delta, out=None, rows=None, n_rows=None):
        self.calls += 1
        if delta is not None:
            residual += delta
        return residual.clone()


class DeferrableNorm(PlainNorm):
    def deferred(self):
        return torch.ones(4), 4, 1e-5


class OldStyleMixer(Mixer):
    """Knows nothing of the protocol: a `then` argument would be a TypeError."""

    def forward(self, h, ctx, cache, write_cache=True):
        assert isinstance(h, torch.Tensor)
        return torch.ones_like(h)


class OldStyleFFN(FeedForward):
    def forward(self, h, ctx):
        assert isinstance(h, torch.Tensor)
        return 2 * torch.ones_like(h)


class NewMixer(Mixer):
    adds_to_residual = True

    def __init__(self, accepts=True, fuses=True):
        self.accepts, self.fuses, self.seen_then, self.seen_owed = accepts, fuses, [], []

    def accepts_owed_norm(self, n_rows):
        return self.accepts

    def forward(self, h, ctx, cache, write_cache=True, then=None):
        self.seen_then.append(then)
        self.seen_owed.append(isinstance(h, OwedNorm))
        x = h.x if isinstance(h, OwedNorm) else h
        if then is not None and self.fuses:
            residual, norm = then
            residual += torch.ones_like(x)
            return OwedNorm(residual.clone(), torch.zeros(x.shape[0], 1), 4, 1e-5, norm)
        return torch.ones_like(x)


class NewFFN(FeedForward):
    adds_to_residual = True

    def __init__(self, accepts=True):
        self.accepts, self.seen_then, self.seen_owed = accepts, [], []

    def accepts_owed_norm(self, n_rows):
        return self.accepts

    def forward(self, h, ctx, then=None):
        self.seen_then.append(then)
        self.seen_owed.append(isinstance(h, OwedNorm))
        x = h.x if isinstance(h, OwedNorm) else h
        if then is not None:
            residual, norm = then
            residual += 2 * torch.ones_like(x)
            return OwedNorm(residual.clone(), torch.zeros(x.shape[0], 1), 4, 1e-5, norm)
        return 2 * torch.ones_like(x)


def stream():
    return HiddenStream(torch.zeros(3, 4))


def test_parts_without_the_protocol_are_run_as_before():
    n1, n2 = DeferrableNorm(), DeferrableNorm()
    block = PreNormBlock(n1, OldStyleMixer(), n2, OldStyleFFN())
    s = stream()
    s.next_norm = DeferrableNorm()          # even when the model offers a reader
    block.forward(s, Ctx(), None)
    assert block.first_norm(3) is None
    assert n1.calls == 1 and n2.calls == 1 and s.owed is None
    assert torch.equal(s.residual, torch.ones(3, 4)) and torch.equal(s.delta, 2 * torch.ones(3, 4))


def test_both_sides_agree_and_the_norms_between_them_do_not_run():
    n1, n2, nxt = DeferrableNorm(), DeferrableNorm(), DeferrableNorm()
    mixer, ffn = NewMixer(), NewFFN()
    block = PreNormBlock(n1, mixer, n2, ffn)
    assert block.first_norm(3) is n1
    s = stream()
    s.next_norm = nxt
    block.forward(s, Ctx(), None)
    assert n1.calls == 1 and n2.calls == 0          # the first norm had nothing prepared, the second was owed
    assert mixer.seen_then[0][1] is n2 and ffn.seen_then[0][1] is nxt
    assert ffn.seen_owed == [True] and mixer.seen_owed == [False]
    assert s.owed is not None and s.owed.norm is nxt and s.delta is None and s.next_norm is None
    assert torch.equal(s.residual, 3 * torch.ones(3, 4))
    # the next block takes the prepared rows instead of running its norm
    block2 = PreNormBlock(nxt, NewMixer(), DeferrableNorm(), NewFFN())
    block2.forward(s, Ctx(), None)
    assert nxt.calls == 0 and block2.mixer.seen_owed == [True]


def test_no_offer_where_the_reader_or_the_norm_says_no():
    # the feed-forward does not take prepared rows: the mixer is not offered the norm between them
    mixer = NewMixer()
    block = PreNormBlock(DeferrableNorm(), mixer, DeferrableNorm(), NewFFN(accepts=False))
    s = stream()
    block.forward(s, Ctx(), None)
    assert mixer.seen_then == [None] and block.norm2.calls == 1
    # a norm that cannot be deferred is never offered
    mixer = NewMixer()
    block = PreNormBlock(PlainNorm(), mixer, PlainNorm(), NewFFN())
    assert block.first_norm(3) is None
    s = stream()
    s.next_norm = None
    block.forward(s, Ctx(), None)
    assert mixer.seen_then == [None] and block.ffn.seen_then == [None]
    # a part that is offered the norm may still answer with a plain delta
    mixer = NewMixer(fuses=False)
    block = PreNormBlock(DeferrableNorm(), mixer, DeferrableNorm(), NewFFN())
    s = stream()
    block.forward(s, Ctx(), None)
    assert mixer.seen_then[0] is not None and block.norm2.calls == 1 and block.ffn.seen_owed == [False]


def test_rows_prepared_for_another_norm_are_refused():
    block = PreNormBlock(DeferrableNorm(), NewMixer(), DeferrableNorm(), NewFFN())
    s = stream()
    s.owed = OwedNorm(torch.zeros(3, 4), torch.zeros(3, 1), 4, 1e-5, DeferrableNorm())
    with pytest.raises(RuntimeError, match="another norm"):
        block.forward(s, Ctx(), None)
