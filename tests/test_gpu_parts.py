"""Each part alone against the plain implementation's function for it."""
import numpy as np
import pytest
import torch

import plain_llama as plain
from helpers import PartHarness, load_part

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 4e-2}


def opts(dtype, max_positions=1024):
    from alpacca_b200.parts import BuildOptions
    return BuildOptions(dtype=DT[dtype], device="cuda", max_positions=max_positions)


def dev(x, dtype):
    return torch.tensor(np.asarray(x)).to(DT[dtype]).cuda()


def rounded(x, dtype):
    """What the part actually sees of an input."""
    return dev(x, dtype).double().cpu().numpy()


def close(got, want, dtype, what=""):
    got = got.double().cpu().numpy() if hasattr(got, "cpu") else np.asarray(got)
    err = np.abs(got - want).max()
    assert err <= TOL[dtype] * max(1.0, np.abs(want).max()), f"{what}: max err {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from alpacca_b200.parts import RMSNorm
    rng = np.random.default_rng(0)
    norm = RMSNorm(opts(dtype), 200, 3e-6, "n")
    w = load_part(norm, 1, dtype)
    res = rng.standard_normal((9, 200)).astype(np.float32)
    delta = rng.standard_normal((9, 200))
    r = torch.tensor(res).cuda()
    got = norm.forward(r, dev(delta, dtype))
    x = res.astype(np.float64) + rounded(delta, dtype)
    close(got, plain.rmsnorm(x, w["n.weight"], 3e-6), dtype)
    close(r, x, "float32", "the residual holds the sum")


@pytest.mark.parametrize("scaling", [None, {"rope_type": "linear", "factor": 2.0},
                                     {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                                      "high_freq_factor": 4.0, "original_max_position_embeddings": 64}])
def test_rotary_tables(scaling):
    from alpacca_b200.parts import RotaryEncoding
    rope = RotaryEncoding(opts("float32", 300), 48, 32, 500000.0, "neox", scaling)
    inv = plain.scale_inv_freq(plain.rope_inv_freq(32, 500000.0), scaling)
    ang = np.arange(300)[:, None] * inv[None, :]
    cos, sin, n_rot, pairing = rope.rotation()
    assert n_rot == 32 and pairing == 1 and cos.shape == (300, 16)
    assert np.abs(cos.cpu().numpy() - np.cos(ang)).max() < 1e-7 and np.abs(sin.cpu().numpy() - np.sin(ang)).max() < 1e-7
    with pytest.raises(ValueError):
        RotaryEncoding(opts("float32"), 48, 50, 1e4, "neox")
    with pytest.raises(ValueError):
        RotaryEncoding(opts("float32"), 48, 32, 1e4, "gptj")


def plain_attention_part(w, prefix, x, H, K, D, n_rot, theta, pairing, scaling, bias, window=None):
    T = len(x)
    pos = np.arange(T)
    inv = plain.scale_inv_freq(plain.rope_inv_freq(n_rot, theta), scaling)
    b = (lambda n: w[f"{prefix}.{n}.bias"]) if bias else (lambda n: None)
    q = plain.rope(plain.linear(x, w[f"{prefix}.q_proj.weight"], b("q_proj")), pos, H, D, n_rot, inv, pairing)
    k = plain.rope(plain.linear(x, w[f"{prefix}.k_proj.weight"], b("k_proj")), pos, K, D, n_rot, inv, pairing)
    v = plain.linear(x, w[f"{prefix}.v_proj.weight"], b("v_proj")).reshape(T, K, D)
    att = plain.attention(q, k, v, window).reshape(T, H * D)
    return plain.linear(att, w[f"{prefix}.o_proj.weight"], b("o_proj"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,K,D,n_rot,pairing,bias,window", [(4, 4, 16, 16, "llama", False, None),
                                                             (6, 2, 32, 32, "neox", True, None),
                                                             (10, 5, 48, 32, "neox", False, 40),
                                                             (3, 1, 24, 12, "llama", True, None)])
def test_attention_part(dtype, H, K, D, n_rot, pairing, bias, window):
    """Two sequences, each fed in two unequal steps and then token by token."""
    from alpacca_b200.parts import Attention, RotaryEncoding
    E, theta = 72, 25000.0
    o = opts(dtype)
    rope = RotaryEncoding(o, D, n_rot, theta, pairing)
    att = Attention(o, E, H, K, D, rope, "a", qkv_bias=bias, out_bias=bias, window=window)
    w = load_part(att, 3, dtype, std=0.15)
    hz = PartHarness([att.cache_spec()], dtype)
    rng = np.random.default_rng(1)
    xs = [rng.standard_normal((n, E)) for n in (70, 133)]
    want = [plain_attention_part(w, "a", rounded(x, dtype), H, K, D, n_rot, theta, pairing, None, bias, window)
            for x in xs]
    slots = [hz.cache.alloc_slot() for _ in xs]
    fed = [0, 0]
    for cuts in ((5, 64), (60, 65), (1, 1), (1, 1), (3, 2)):
        ctx = hz.step(list(zip(slots, cuts)))
        h = torch.cat([dev(x[f:f + c], dtype) for x, f, c in zip(xs, fed, cuts)])
        got = att.forward(h, ctx, hz.cache.entry_view(0, ctx.block_tables))
        hz.done()
        at = 0
        for i, c in enumerate(cuts):
            close(got[at:at + c], want[i][fed[i]:fed[i] + c], dtype, f"seq {i} rows {fed[i]}..{fed[i] + c}")
            at += c
            fed[i] += c


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [1, 5, 40])
def test_swiglu_part(dtype, T):
    from alpacca_b200.parts import SwiGLU
    from types import SimpleNamespace
    ffn = SwiGLU(opts(dtype), 72, 264, "m", bias=True)
    w = load_part(ffn, 5, dtype, std=0.2)
    x = np.random.default_rng(2).standard_normal((T, 72))
    got = ffn.forward(dev(x, dtype), SimpleNamespace(n_tokens=T))
    xr = rounded(x, dtype)
    a = plain.swiglu(plain.linear(xr, w["m.gate_proj.weight"], w["m.gate_proj.bias"]),
                     plain.linear(xr, w["m.up_proj.weight"], w["m.up_proj.bias"]))
    close(got, plain.linear(a, w["m.down_proj.weight"], w["m.down_proj.bias"]), dtype)
    with pytest.raises(ValueError, match="multiple of 8"):
        SwiGLU(opts(dtype), 72, 100, "m")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head(dtype):
    from alpacca_b200.parts import TokenEmbedding, VocabHead
    o = opts(dtype)
    emb = TokenEmbedding(o, 1003, 72, "e")
    w = load_part(emb, 6, dtype)
    toks = torch.tensor([0, 1002, 17, 17], dtype=torch.int32).cuda()
    x = emb.forward(toks, 4)
    assert x.dtype == torch.float32
    close(x, w["e.weight"][[0, 1002, 17, 17]], "float32")
    h = np.random.default_rng(3).standard_normal((20, 72))
    tied = VocabHead(o, 1003, 72, "lm_head", tied_to=emb)
    assert [s.absent for s in tied.param_specs()] == [True]
    logits = tied.forward(dev(h, dtype))
    assert logits.dtype == torch.float32
    close(logits, plain.linear(rounded(h, dtype), w["e.weight"]), dtype)
    untied = VocabHead(o, 1003, 72, "lm_head")
    w2 = load_part(untied, 7, dtype)
    close(untied.forward(dev(h[:3], dtype)), plain.linear(rounded(h[:3], dtype), w2["lm_head.weight"]), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block(dtype):
    """A whole pre-norm block: x += Attn(norm1 x); x += FFN(norm2 x)."""
    from alpacca_b200.parts import Attention, HiddenStream, PreNormBlock, RMSNorm, RotaryEncoding, SwiGLU
    E, H, K, D = 72, 6, 3, 16
    o = opts(dtype)
    blk = PreNormBlock(RMSNorm(o, E, 1e-5, "n1"), Attention(o, E, H, K, D, RotaryEncoding(o, D, D, 1e4, "neox"), "a"),
                       RMSNorm(o, E, 1e-5, "n2"), SwiGLU(o, E, 160, "m"))
    w = load_part(blk, 8, dtype, std=0.15)
    for n in ("n1.weight", "n2.weight"):
        assert abs(w[n].mean() - 1) < 0.2
    hz = PartHarness([blk.mixer.cache_spec()], dtype)
    x = np.random.default_rng(4).standard_normal((50, E)).astype(np.float32)
    slot = hz.cache.alloc_slot()
    ctx = hz.step([(slot, 50)])
    stream = HiddenStream(torch.tensor(x).cuda())
    blk.forward(stream, ctx, hz.cache.entry_view(0, ctx.block_tables))
    got = stream.residual.double().cpu().numpy() + stream.delta.double().cpu().numpy()
    xd = x.astype(np.float64)
    a = plain_attention_part(w, "a", plain.rmsnorm(xd, w["n1.weight"], 1e-5), H, K, D, D, 1e4, "neox", None, False)
    y = xd + a
    hn = plain.rmsnorm(y, w["n2.weight"], 1e-5)
    y = y + plain.linear(plain.swiglu(plain.linear(hn, w["m.gate_proj.weight"]), plain.linear(hn, w["m.up_proj.weight"])),
                         w["m.down_proj.weight"])
    close(got, y, dtype)


def test_timers_attribute_device_time_to_operations(model_dirs):
    """`ops.timers()`: a prompt step issued launch by launch gives a time for every kind of operation
    that ran, and nothing is recorded outside the `with`."""
    import tiny
    from alpacca_b200 import ops
    from alpacca_b200.engine import Engine, StepEntry
    from alpacca_b200.engine.loading import load_model_dir
    eng = Engine(load_model_dir(model_dirs[("d", "bfloat16")], dtype="bfloat16"), max_tokens=64 * 8, max_slots=2)
    toks = tiny.prompt_tokens(tiny.TINY_D, 200, 5)
    slot = eng.alloc_slot()
    with ops.timers() as t:
        eng.step([StepEntry(slot, toks, [199])])
    tot = t.totals()
    assert {"embed_rows", "add_rmsnorm", "rope_append", "library product"} <= set(tot), tot
    assert any(k.startswith("attention") for k in tot) and all(us > 0 for _, us in tot.values())
    assert tot["add_rmsnorm"][0] == 2 * 2 + 1 and "total" in t.table()
    n = len(t.marks)
    eng.step([StepEntry(slot, [toks[0]], [0])])
    assert len(t.marks) == n and ops._timeline is None
