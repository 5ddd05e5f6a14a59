"""Parts of other kinds, defined here and nowhere in the package, put together into a model by
configuration: a feed-forward with routed experts, a position encoding that adds a learned term to the
embeddings (and attention without rotation), a norm that centres, a block that runs mixer and
feed-forward side by side, and layers that differ (one with a window, so its keys have storage of
their own).  None of it is anyone's model: it shows that the package's interfaces carry such parts
without a change to its files."""
from dataclasses import dataclass
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu

NAME = "ToyRoutedForCausalLM"
TOY = {"architectures": [NAME], "width": 48, "heads": 3, "kv_heads": 3, "head_dim": 16, "inner": 40, "experts": 5,
       "experts_per_token": 2, "vocab": 83, "eps": 1e-5, "positions": 200, "window": 24, "eos_token_id": 82}


def define_toy():
    from alpacca_b200.config import ModelConfig, register_architecture, unregister_architecture
    from alpacca_b200.engine.model import DecoderSpec
    from alpacca_b200.parts import (Attention, FeedForward, Norm, Part, PositionEncoding, PreNormBlock, RMSNorm,
                                    SwiGLU, TokenEmbedding, VocabHead)
    from alpacca_b200.weights import ParamSpec

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        width: int = 32
        heads: int = 2
        kv_heads: int = 2
        head_dim: int = 16
        inner: int = 32
        experts: int = 4
        experts_per_token: int = 2
        vocab: int = 50
        eps: float = 1e-5
        positions: int = 128
        window: int = 16
        eos_token_id: int = 0

        # what architecture-neutral code asks of a configuration, answered from this one's own keys
        @property
        def max_positions(self):
            return self.positions

        @property
        def stop_tokens(self):
            return (self.eos_token_id,)

    class LearnedPositions(PositionEncoding):
        """x_t += table[position of t]; nothing is rotated."""

        def __init__(self, opts, positions, width, name):
            self.opts, self.positions, self.width, self.name = opts, positions, width, name
            self.table = None

        def own_param_specs(self):
            return [ParamSpec(f"{self.name}.weight", (self.positions, self.width), "keep32", "normal")]

        def load_own(self, fetch):
            self.table = fetch(self.own_param_specs()[0])

        def add_to_embeddings(self, residual, ctx):
            T = ctx.n_tokens
            residual[:T] += self.table[ctx.tok_pos[:T].long()].float()

    class CentredNorm(Norm):
        """y = (x - mean) / sqrt(var + eps) * w, with the pending output added to the stream first."""

        def __init__(self, opts, width, eps, name):
            self.opts, self.width, self.eps, self.name = opts, width, eps, name
            self.weight = None

        def own_param_specs(self):
            return [ParamSpec(f"{self.name}.weight", (self.width,), "vector", "one_plus_normal")]

        def load_own(self, fetch):
            self.weight = fetch(self.own_param_specs()[0])

        def forward(self, residual, delta, out=None, rows=None, n_rows=None):
            if rows is not None:
                x = residual[rows[:n_rows].long()]
                if delta is not None:
                    x = x + delta[rows[:n_rows].long()].float()
            else:
                if delta is not None:
                    residual += delta.float()
                x = residual
            x = x - x.mean(-1, keepdim=True)
            return (x / torch.sqrt((x * x).mean(-1, keepdim=True) + self.eps) * self.weight).to(self.opts.dtype)

    class RoutedFFN(FeedForward):
        """Every token goes to its `top` best experts by (router logit + a step that depends on the token
        id and the expert); their outputs are added with the softmax of their router logits as weights.
        The step, multiples of 32, makes the choice clear-cut, so that rounding cannot tip it; the weights
        still follow the activations.  The router is float32."""
        graph_capturable = False      # which rows go where is read on the host

        def __init__(self, opts, width, inner, n_experts, top, prefix):
            self.opts, self.top, self.prefix, self.width, self.n_experts = opts, top, prefix, width, n_experts
            self.experts = [SwiGLU(opts, width, inner, f"{prefix}.experts.{e}") for e in range(n_experts)]
            self.router = None

        def own_param_specs(self):
            return [ParamSpec(f"{self.prefix}.router.weight", (self.n_experts, self.width), "keep32", "normal")]

        def load_own(self, fetch):
            self.router = fetch(self.own_param_specs()[0])

        def forward(self, h, ctx):
            T = ctx.n_tokens
            logits = h[:T].float() @ self.router.float().T
            e = torch.arange(self.n_experts, device=h.device)
            step = 32.0 * ((2 * ctx.tokens[:T].long().unsqueeze(-1) + 3 * e) % self.n_experts)
            _, idx = torch.topk(logits + step, self.top, dim=-1)
            gate = torch.softmax(torch.gather(logits, 1, idx), dim=-1)
            out = torch.zeros((h.shape[0], self.width), dtype=torch.float32, device=h.device)
            for e, expert in enumerate(self.experts):
                tok, which = torch.nonzero(idx == e, as_tuple=True)
                if tok.numel() == 0:
                    continue
                y = expert.forward(h[tok].contiguous(), SimpleNamespace(n_tokens=int(tok.numel())))[:tok.numel()]
                out.index_add_(0, tok, y.float() * gate[tok, which].unsqueeze(-1))
            return out.to(h.dtype)

    class SideBySideBlock(Part):
        """x += Mixer(Norm(x)) + FeedForward(Norm(x)): one norm, both sub-layers read it."""

        def __init__(self, norm, mixer, ffn):
            self.norm, self.mixer, self.ffn = norm, mixer, ffn

        def forward(self, stream, ctx, cache, write_cache=True):
            h = self.norm.forward(stream.residual, stream.delta)
            a = self.mixer.forward(h, ctx, cache, write_cache)
            f = self.ffn.forward(h, ctx)
            stream.delta = (a.float() + f.float()).to(a.dtype)

    unregister_architecture(NAME)

    @register_architecture(NAME, ToyConfig)
    def build(cfg, opts):
        E = cfg.width
        emb = TokenEmbedding(opts, cfg.vocab, E, "emb")
        layers = [
            PreNormBlock(RMSNorm(opts, E, cfg.eps, "l0.n1"),
                         Attention(opts, E, cfg.heads, cfg.kv_heads, cfg.head_dim, None, "l0.attn"),
                         RMSNorm(opts, E, cfg.eps, "l0.n2"),
                         RoutedFFN(opts, E, cfg.inner, cfg.experts, cfg.experts_per_token, "l0.moe")),
            SideBySideBlock(CentredNorm(opts, E, cfg.eps, "l1.n"),
                            Attention(opts, E, cfg.heads, 1, cfg.head_dim, None, "l1.attn", window=cfg.window),
                            SwiGLU(opts, E, cfg.inner, "l1.ffn")),
        ]
        return DecoderSpec(embedding=emb, layers=layers, final_norm=CentredNorm(opts, E, cfg.eps, "norm"),
                           head=VocabHead(opts, cfg.vocab, E, "head", tied_to=emb),
                           position=LearnedPositions(opts, cfg.positions, E, "pos"),
                           stop_token_ids=(cfg.eos_token_id,), vocab_size=cfg.vocab)
    return ToyConfig


def plain_toy(cfg, w, tokens):
    """Whole sequence, float64, no cache."""
    E, H, D, top = cfg["width"], cfg["heads"], cfg["head_dim"], cfg["experts_per_token"]
    T = len(tokens)
    x = plain.embed(w["emb.weight"], tokens) + w["pos.weight"][:T].astype(np.float64)

    def centred(x, weight):
        c = x - x.mean(-1, keepdims=True)
        return c / np.sqrt((c * c).mean(-1, keepdims=True) + cfg["eps"]) * weight

    def swiglu_ffn(h, p):
        a = plain.swiglu(plain.linear(h, w[p + ".gate_proj.weight"]), plain.linear(h, w[p + ".up_proj.weight"]))
        return plain.linear(a, w[p + ".down_proj.weight"])

    def attend(h, p, kv_heads, window):
        q = plain.linear(h, w[p + ".q_proj.weight"]).reshape(T, H, D)
        k = plain.linear(h, w[p + ".k_proj.weight"]).reshape(T, kv_heads, D)
        v = plain.linear(h, w[p + ".v_proj.weight"]).reshape(T, kv_heads, D)
        return plain.linear(plain.attention(q, k, v, window=window).reshape(T, H * D), w[p + ".o_proj.weight"])

    # layer 0: attention without rotation, then routed experts
    x = x + attend(plain.rmsnorm(x, w["l0.n1.weight"], cfg["eps"]), "l0.attn", cfg["kv_heads"], None)
    h = plain.rmsnorm(x, w["l0.n2.weight"], cfg["eps"])
    logits = h @ w["l0.moe.router.weight"].astype(np.float64).T
    step = 32.0 * ((2 * np.asarray(tokens)[:, None] + 3 * np.arange(cfg["experts"])) % cfg["experts"])
    assert np.abs(logits).max() < 12.0, "the step of 32 must decide the choice"
    y = np.zeros_like(x)
    for t in range(T):
        best = np.argsort(-(logits[t] + step[t]), kind="stable")[:top]
        g = np.exp(logits[t, best] - logits[t, best].max())
        g /= g.sum()
        for e, ge in zip(best, g):
            y[t] += ge * swiglu_ffn(h[t:t + 1], f"l0.moe.experts.{e}")[0]
    x = x + y
    # layer 1: mixer and feed-forward side by side on one centred norm, a window of keys, one KV head
    h = centred(x, w["l1.n.weight"])
    x = x + attend(h, "l1.attn", 1, cfg["window"]) + swiglu_ffn(h, "l1.ffn")
    return plain.linear(centred(x, w["norm.weight"]), w["emb.weight"])


@pytest.fixture(scope="module")
def toy_dir(tmp_path_factory):
    define_toy()
    from alpacca_b200.engine.loading import write_random_model_dir
    d = write_random_model_dir(tmp_path_factory.mktemp("toy_parts"), TOY, seed=9, dtype="float32", std=0.2)
    yield d
    from alpacca_b200.config import unregister_architecture
    unregister_architecture(NAME)


def test_layers_of_different_parts_get_storage_of_their_own(toy_dir):
    from alpacca_b200.engine import Engine
    from alpacca_b200.engine.loading import load_model_dir
    model = load_model_dir(toy_dir, dtype="float32")
    specs = model.cache_entry_specs()
    assert [(s.n_kv_heads, s.window) for s in specs] == [(3, None), (1, 24)]
    eng = Engine(model, max_tokens=64 * 6, max_slots=2)
    assert len(eng.cache.kv_groups) == 2, "all keys and a window of keys are two groups"
    names = {s.name for s in model.param_specs() if not s.absent}
    assert set(plain.read_safetensors(toy_dir / "model.safetensors")) == names
    assert "l0.moe.experts.4.down_proj.weight" in names and "pos.weight" in names


@pytest.mark.parametrize("dtype,rel", [("float32", 5e-5), ("bfloat16", 4e-2)])
def test_stepped_whole_one_by_one_and_in_batches(toy_dir, dtype, rel):
    from alpacca_b200.engine import Engine, StepEntry
    from alpacca_b200.engine.loading import load_model_dir
    cfg, w = plain.read_model_dir(toy_dir)
    eng = Engine(load_model_dir(toy_dir, dtype=dtype), max_tokens=64 * 8, max_slots=3)
    rng = np.random.default_rng(1)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (90, 7, 41)]
    want = [plain_toy(cfg, w, s) for s in seqs]
    tol = rel * max(1.0, max(np.abs(x).max() for x in want))
    for round_ in range(2):
        slots = [eng.alloc_slot() for _ in seqs]
        heads = [len(s) - 5 - i for i, s in enumerate(seqs)]
        got = eng.step([StepEntry(sl, s[:h], list(range(h))) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
        at, worst = 0, 0.0
        for i, h in enumerate(heads):
            worst = max(worst, np.abs(got[at:at + h] - want[i][:h]).max())
            at += h
        assert worst < tol, (round_, "whole", worst, tol)
        pos, live = list(heads), [0, 1, 2]
        while live:
            got = eng.step([StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                assert np.abs(got[row] - want[i][pos[i]]).max() < tol, (round_, i, pos[i])
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.free_slot(slots[i])
                live.remove(i)
        eng.cache.check()


def test_generation_through_the_entry_point(toy_dir):
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    cfg, w = plain.read_model_dir(toy_dir)
    model = Model.load(toy_dir, dtype="float32", max_batch=2)
    assert not model.use_graphs          # the routed feed-forward reads on the host: step-by-step decoding
    prompts = [[5, 6, 7, 8], [2] * 30]
    res = generate(model, prompts, SamplerParams.greedy(), n_predict=8, stop_token_ids=[])
    for p, r in zip(prompts, res):
        seq = list(p)
        for t in r.token_ids:
            row = plain_toy(cfg, w, seq)[-1]
            assert row[t] >= row.max() - 1e-4
            seq.append(t)
