"""Another architecture, defined here and nowhere in the package: a mixer with a state of fixed size
per sequence, a layer that runs twice, a run that reads another run's cache, and a layer whose block
holds two mixers that both keep something (keys and values beside a state).  It is registered, built,
given random weights, stepped and generated from without a change to the package's files."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu

TOY = {"architectures": ["ToyDecayForCausalLM"], "n_layers": 2, "width": 40, "state": 24, "heads": 4, "kv_heads": 2,
       "head_dim": 16, "inner": 64, "vocab": 97, "eps": 1e-5, "positions": 256, "eos_token_id": 96}


def define_toy():
    from alpacca_b200.config import ModelConfig, register_architecture, unregister_architecture
    from alpacca_b200.engine.model import DecoderSpec, Run
    from alpacca_b200.parts import (Attention, Block, Linear, Mixer, PreNormBlock, RMSNorm, RotaryEncoding, StateSpec,
                                    SwiGLU, TokenEmbedding, VocabHead)
    from alpacca_b200.weights import ParamSpec

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        n_layers: int = 2
        width: int = 32
        state: int = 16
        heads: int = 4
        kv_heads: int = 2
        head_dim: int = 16
        inner: int = 64
        vocab: int = 50
        eps: float = 1e-5
        positions: int = 256
        eos_token_id: int = 0

        # what architecture-neutral code asks of a configuration, answered from this one's own keys
        @property
        def max_positions(self):
            return self.positions

        @property
        def stop_tokens(self):
            return (self.eos_token_id,)

    class DecayMixer(Mixer):
        """s_t = sigmoid(a) * s_{t-1} + W_in h_t;  y_t = W_out s_t.  The state s lives per sequence."""
        graph_capturable = False      # it walks the batch on the host

        def __init__(self, opts, width, state, prefix):
            self.opts, self.width, self.n_state, self.prefix = opts, width, state, prefix
            self.w_in = Linear(opts, width, [(f"{prefix}.in_proj", state)])
            self.w_out = Linear(opts, state, [(f"{prefix}.out_proj", width)])
            self.decay = None

        def own_param_specs(self):
            return [ParamSpec(f"{self.prefix}.decay", (self.n_state,), "vector", "normal")]

        def load_own(self, fetch):
            self.decay = fetch(self.own_param_specs()[0])

        def cache_spec(self):
            return StateSpec((self.n_state,), torch.float32)

        def forward(self, h, ctx, cache, write_cache=True):
            u = self.w_in.forward(h, n_rows=ctx.n_tokens).float()
            a = torch.sigmoid(self.decay)
            ys = torch.empty_like(u)
            at = 0
            for slot, n in zip(ctx.host_slots, ctx.host_q_lens):
                s = cache.state[slot].clone()
                for t in range(at, at + n):
                    s = a * s + u[t]
                    ys[t] = s
                if write_cache:
                    cache.state[slot] = s
                at += n
            return self.w_out.forward(ys.to(h.dtype), n_rows=ctx.n_tokens)

    class HybridBlock(Block):
        """x += Attention(Norm1(x)) + Decay(Norm1(x)); x += FeedForward(Norm2(x)): two mixers in one
        layer, each with a cache entry of its own (keys and values; a state)."""

        def __init__(self, norm1, attention, decay, norm2, ffn):
            self.norm1, self.attention, self.decay, self.norm2, self.ffn = norm1, attention, decay, norm2, ffn

        def cache_specs(self):
            return [self.attention.cache_spec(), self.decay.cache_spec()]

        def forward(self, stream, ctx, cache, write_cache=True):
            kv, state = cache
            h = self.norm1.forward(stream.residual, stream.delta)
            a = self.attention.forward(h, ctx, kv, write_cache)
            d = self.decay.forward(h, ctx, state, write_cache)
            h = self.norm2.forward(stream.residual, (a.float() + d.float()).to(a.dtype))
            stream.delta = self.ffn.forward(h, ctx)

    unregister_architecture("ToyDecayForCausalLM")

    @register_architecture("ToyDecayForCausalLM", ToyConfig)
    def build(cfg, opts):
        E = cfg.width
        rope = RotaryEncoding(opts, cfg.head_dim, cfg.head_dim, 10000.0, "neox", max_positions=cfg.positions)
        emb = TokenEmbedding(opts, cfg.vocab, E, "emb")
        layers = [
            PreNormBlock(RMSNorm(opts, E, cfg.eps, "l0.n1"), DecayMixer(opts, E, cfg.state, "l0.mix"),
                         RMSNorm(opts, E, cfg.eps, "l0.n2"), SwiGLU(opts, E, cfg.inner, "l0.ffn")),
            PreNormBlock(RMSNorm(opts, E, cfg.eps, "l1.n1"),
                         Attention(opts, E, cfg.heads, cfg.kv_heads, cfg.head_dim, rope, "l1.attn"),
                         RMSNorm(opts, E, cfg.eps, "l1.n2"), SwiGLU(opts, E, cfg.inner, "l1.ffn")),
            HybridBlock(RMSNorm(opts, E, cfg.eps, "l2.n1"),
                        Attention(opts, E, cfg.heads, cfg.kv_heads, cfg.head_dim, rope, "l2.attn"),
                        DecayMixer(opts, E, cfg.state, "l2.mix"),
                        RMSNorm(opts, E, cfg.eps, "l2.n2"), SwiGLU(opts, E, cfg.inner, "l2.ffn")),
        ]
        # layer 0 runs twice (two states), layer 1 runs twice and its second run reads the first one's
        # keys, layer 2 keeps keys and a state at once
        schedule = [Run(0), Run(1), Run(0), Run(1, reads_entry_of=1), Run(2)]
        return DecoderSpec(embedding=emb, layers=layers, final_norm=RMSNorm(opts, E, cfg.eps, "norm"),
                           head=VocabHead(opts, cfg.vocab, E, "head", tied_to=emb), schedule=schedule,
                           stop_token_ids=(cfg.eos_token_id,), vocab_size=cfg.vocab)
    return ToyConfig


def plain_toy(cfg, w, tokens):
    """Whole sequence, float64, no cache."""
    E, H, K, D = cfg["width"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    T = len(tokens)
    x = plain.embed(w["emb.weight"], tokens)
    inv = plain.rope_inv_freq(D, 10000.0)
    pos = np.arange(T)

    def ffn(x, p):
        h = plain.rmsnorm(x, w[p + ".n2.weight"], cfg["eps"])
        a = plain.swiglu(plain.linear(h, w[p + ".ffn.gate_proj.weight"]), plain.linear(h, w[p + ".ffn.up_proj.weight"]))
        return x + plain.linear(a, w[p + ".ffn.down_proj.weight"])

    def decay(h, p):
        u = plain.linear(h, w[p + ".mix.in_proj.weight"])
        a = 1 / (1 + np.exp(-w[p + ".mix.decay"]))
        s, ys = np.zeros(cfg["state"]), []
        for t in range(T):
            s = a * s + u[t]
            ys.append(s)
        return plain.linear(np.stack(ys), w[p + ".mix.out_proj.weight"])

    def attend(h, p, kv=None):
        q = plain.rope(plain.linear(h, w[p + ".attn.q_proj.weight"]), pos, H, D, D, inv, "neox")
        if kv is None:
            k = plain.rope(plain.linear(h, w[p + ".attn.k_proj.weight"]), pos, K, D, D, inv, "neox")
            v = plain.linear(h, w[p + ".attn.v_proj.weight"]).reshape(T, K, D)
            kv = (k, v)
        a = plain.attention(q, kv[0], kv[1]).reshape(T, H * D)
        return plain.linear(a, w[p + ".attn.o_proj.weight"]), kv

    def decay_layer(x):
        return ffn(x + decay(plain.rmsnorm(x, w["l0.n1.weight"], cfg["eps"]), "l0"), "l0")

    def attn_layer(x, kv=None):
        a, kv = attend(plain.rmsnorm(x, w["l1.n1.weight"], cfg["eps"]), "l1", kv)
        return ffn(x + a, "l1"), kv

    def hybrid_layer(x):
        h = plain.rmsnorm(x, w["l2.n1.weight"], cfg["eps"])
        return ffn(x + attend(h, "l2")[0] + decay(h, "l2"), "l2")

    x = decay_layer(x)
    x, kv = attn_layer(x)
    x = decay_layer(x)
    x, _ = attn_layer(x, kv)
    x = hybrid_layer(x)
    return plain.linear(plain.rmsnorm(x, w["norm.weight"], cfg["eps"]), w["emb.weight"])


@pytest.fixture(scope="module")
def toy_dir(tmp_path_factory):
    define_toy()
    from alpacca_b200.engine.loading import write_random_model_dir
    d = write_random_model_dir(tmp_path_factory.mktemp("toy"), TOY, seed=4, dtype="float32", std=0.2)
    yield d
    from alpacca_b200.config import unregister_architecture
    unregister_architecture("ToyDecayForCausalLM")


def test_registered_built_and_loaded(toy_dir):
    from alpacca_b200.config import registered_architectures
    from alpacca_b200.engine.loading import load_model_dir
    assert "ToyDecayForCausalLM" in registered_architectures()
    model = load_model_dir(toy_dir, dtype="float32")
    specs = model.cache_entry_specs()
    assert [type(s).__name__ for s in specs] == ["StateSpec", "KVSpec", "StateSpec", "KVSpec", "StateSpec"]
    # the fourth run reads the second run's entry; the last run's block keeps two things
    assert model.entries_of_run == [[0], [1], [2], [1], [3, 4]] and not model.all_capturable()
    names = {s.name for s in model.param_specs() if not s.absent}
    assert set(plain.read_safetensors(toy_dir / "model.safetensors")) == names


@pytest.mark.parametrize("dtype,rel", [("float32", 5e-5), ("bfloat16", 4e-2)])
def test_stepped_whole_one_by_one_and_in_batches(toy_dir, dtype, rel):
    from alpacca_b200.engine import Engine, StepEntry
    from alpacca_b200.engine.loading import load_model_dir
    cfg, w = plain.read_model_dir(toy_dir)
    eng = Engine(load_model_dir(toy_dir, dtype=dtype), max_tokens=64 * 8, max_slots=3)
    assert len(eng.cache.state_groups) == 1 and eng.cache.state_groups[0].state.shape[:2] == (3, 3)
    assert len(eng.cache.kv_groups) == 1 and eng.cache.kv_groups[0].n_entries == 2
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (70, 9, 33)]
    want = [plain_toy(cfg, w, s) for s in seqs]
    # the same share of the logits' magnitude as the tolerances of the Llama tests (logits of order 1 there)
    tol = rel * max(1.0, max(np.abs(x).max() for x in want))
    for round_ in range(2):                     # the second round reuses slots and their state rows
        slots = [eng.alloc_slot() for _ in seqs]
        heads = [len(s) - 4 - i for i, s in enumerate(seqs)]
        got = eng.step([StepEntry(sl, s[:h], [0, h - 1]) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
        for i, h in enumerate(heads):
            assert np.abs(got[2 * i] - want[i][0]).max() < tol and np.abs(got[2 * i + 1] - want[i][h - 1]).max() < tol
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


def test_generation_falls_back_to_stepwise_decoding(toy_dir):
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    cfg, w = plain.read_model_dir(toy_dir)
    model = Model.load(toy_dir, dtype="float32", max_batch=2)
    assert not model.use_graphs
    prompts = [[5, 6, 7], [1] * 20]
    res = generate(model, prompts, SamplerParams.greedy(), n_predict=6, stop_token_ids=[])
    for p, r in zip(prompts, res):
        seq = list(p)
        for t in r.token_ids:
            row = plain_toy(cfg, w, seq)[-1]
            assert row[t] >= row.max() - 1e-4
            seq.append(t)
