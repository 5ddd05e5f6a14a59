"""Each kernel alone against a plain float32/float64 reference of the same operation,
at sizes other than the engine's: widths and vocabularies that are no power of two,
head sizes in steps of 16, several heads-per-group ratios."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# relative to the magnitude of the outputs (order 1 here): float32 sums of a few hundred
# terms; bfloat16 results rounded once to 8 bits of mantissa
TOL = {"float32": 2e-5, "bfloat16": 1.6e-2}


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).cuda()


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item()
    mag = max(want.abs().max().item(), 1.0)
    assert math.isfinite(err) and err <= TOL[dtype] * mag, f"{what}: max err {err:.3e} (magnitude {mag:.2f})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("V,E", [(300, 72), (1003, 200)])
def test_embed_rows(dtype, V, E):
    from alpacca_b200 import ops
    table = rnd(V, E, dtype=DT[dtype])
    toks = torch.tensor([0, V - 1, 5, 5, 17], dtype=torch.int32).cuda()
    out = torch.empty(5, E, dtype=torch.float32, device="cuda")
    ops.embed_rows(table, toks, out)
    assert torch.equal(out, table[toks.long()].float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,eps", [(1, 72, 1e-5), (7, 200, 1e-6), (33, 2056, 3e-6)])
def test_add_rmsnorm(dtype, T, E, eps):
    from alpacca_b200 import ops
    res = rnd(T, E, seed=1)
    delta = rnd(T, E, dtype=DT[dtype], seed=2)
    w = 1 + rnd(E, seed=3) * 0.1
    want_res = res.double() + delta.double()
    want = want_res / torch.sqrt((want_res ** 2).mean(-1, keepdim=True) + eps) * w.double()
    r = res.clone()
    out = torch.empty(T, E, dtype=DT[dtype], device="cuda")
    ops.add_rmsnorm(r, delta, w, eps, out)
    close(out, want, dtype, "normed")
    close(r, want_res, "float32", "residual after the add")
    # rows: picked rows only, residual untouched
    rows = torch.tensor([T - 1, 0], dtype=torch.int32).cuda()
    r2 = res.clone()
    out2 = torch.empty(2, E, dtype=DT[dtype], device="cuda")
    ops.add_rmsnorm(r2, delta, w, eps, out2, rows=rows)
    close(out2, want[[T - 1, 0]], dtype, "picked rows")
    assert torch.equal(r2, res)
    # without delta
    out3 = torch.empty(T, E, dtype=DT[dtype], device="cuda")
    ops.add_rmsnorm(res.clone(), None, w, eps, out3)
    want3 = res.double() / torch.sqrt((res.double() ** 2).mean(-1, keepdim=True) + eps) * w.double()
    close(out3, want3, dtype, "no delta")


def ref_rope(x, pos, n_rot, pairing, cos, sin):
    """x [T, heads, D] float64."""
    x = x.clone()
    half = n_rot // 2
    c, s = cos[pos][:, None, :].double(), sin[pos][:, None, :].double()
    if pairing == 0:
        a, b = x[..., 0:n_rot:2].clone(), x[..., 1:n_rot:2].clone()
        x[..., 0:n_rot:2], x[..., 1:n_rot:2] = a * c - b * s, a * s + b * c
    else:
        a, b = x[..., :half].clone(), x[..., half:n_rot].clone()
        x[..., :half], x[..., half:n_rot] = a * c - b * s, a * s + b * c
    return x


def make_paged(lengths, n_pages, K, D, dtype, page=64, seed=0):
    """Block table with pages handed out in a scattered order; returns table, k/v pages."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // page) for n in lengths)
    table = torch.zeros(len(lengths), width, dtype=torch.int32)
    for b, n in enumerate(lengths):
        for i in range(-(-n // page)):
            table[b, i] = perm.pop()
    k = torch.zeros(n_pages, K, page, D, dtype=dtype, device="cuda")
    v = torch.zeros_like(k)
    return table.cuda(), k, v


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,K,D,n_rot,pairing", [(4, 4, 16, 16, 0), (6, 2, 32, 32, 1), (10, 5, 48, 32, 1),
                                                 (3, 1, 80, 40, 0)])
def test_rope_append(dtype, H, K, D, n_rot, pairing):
    from alpacca_b200 import ops
    lengths = [70, 3, 130]           # tokens already there + new ones; new tokens are the last q_len
    q_lens = [5, 3, 66]
    table, kp, vp = make_paged(lengths, 8, K, D, DT[dtype])
    T = sum(q_lens)
    qkv = rnd(T, (H + 2 * K) * D, dtype=DT[dtype], seed=5)
    pos = torch.cat([torch.arange(n - q, n) for n, q in zip(lengths, q_lens)]).to(torch.int32)
    seq = torch.cat([torch.full((q,), b) for b, q in enumerate(q_lens)]).to(torch.int32)
    P = 160
    inv = 10000.0 ** (-torch.arange(n_rot // 2, dtype=torch.float64) * 2 / n_rot)
    ang = torch.arange(P, dtype=torch.float64)[:, None] * inv
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    x = qkv.double().cpu().view(T, H + 2 * K, D)
    want_qk = ref_rope(x[:, :H + K], pos.long(), n_rot, pairing, cos.cpu(), sin.cpu())
    got = qkv.clone()
    ops.rope_append(got, cos, sin, pos.cuda(), seq.cuda(), table, kp, vp, T, H, K, D, n_rot, pairing)
    g = got.double().cpu().view(T, H + 2 * K, D)
    close(g[:, :H], want_qk[:, :H], dtype, "q rotated in place")
    tb = table.cpu()
    for t in range(T):
        page, off = tb[seq[t], pos[t] // 64].item(), pos[t].item() % 64
        close(kp[page, :, off], want_qk[t, H:], dtype, f"k of token {t} in the cache")
        close(vp[page, :, off], x[t, H + K:], dtype, f"v of token {t} in the cache")
    # padding tokens are skipped
    got2, kp2 = qkv.clone(), torch.zeros_like(kp)
    ops.rope_append(got2, cos, sin, pos.cuda(), torch.full_like(seq, -1).cuda(), table, kp2, torch.zeros_like(vp),
                    T, H, K, D, n_rot, pairing)
    assert torch.equal(got2, qkv) and kp2.abs().sum().item() == 0


def ref_attention(q, k, v, pos_q, scale, window=0):
    """q [Tq,H,D], k/v [S,K,D] float64, pos_q: position of each query."""
    Tq, H, D = q.shape
    G = H // k.shape[1]
    out = torch.zeros(Tq, H, D, dtype=torch.float64)
    for t in range(Tq):
        p = int(pos_q[t])
        lo = max(0, p - window + 1) if window else 0
        for h in range(H):
            sc = (k[lo:p + 1, h // G] @ q[t, h]) * scale
            out[t, h] = torch.softmax(sc, 0) @ v[lo:p + 1, h // G]
    return out


def fill_cache(table, kp, vp, b, kk, vv):
    for s in range(kk.shape[0]):
        page = table[b, s // 64].item()
        kp[page, :, s % 64] = kk[s].to(kp.dtype)
        vp[page, :, s % 64] = vv[s].to(vp.dtype)


ATT_CASES = [(4, 4, 16), (6, 2, 32), (10, 5, 48), (8, 1, 64), (5, 5, 80), (4, 2, 128), (2, 1, 256), (14, 2, 96)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,K,D", ATT_CASES)
@pytest.mark.parametrize("window", [0, 37])
def test_attention_prefill_and_decode(dtype, H, K, D, window):
    """Three sequences in one launch: a prompt from position 0, a chunk on top of cached
    tokens, and a single decode token far into its sequence."""
    from alpacca_b200 import ops
    from alpacca_b200.cache import KVLayerView
    from types import SimpleNamespace
    lengths, q_lens = [75, 200, 301], [75, 40, 1]
    table, kp, vp = make_paged(lengths, 12, K, D, DT[dtype], seed=D)
    T = sum(q_lens)
    qkv = rnd(T, (H + 2 * K) * D, dtype=DT[dtype], seed=7)
    ks = [rnd(n, K, D, dtype=DT[dtype], seed=8 + b) for b, n in enumerate(lengths)]
    vs = [rnd(n, K, D, dtype=DT[dtype], seed=11 + b) for b, n in enumerate(lengths)]
    for b in range(3):
        fill_cache(table.cpu(), kp, vp, b, ks[b], vs[b])
    pos = torch.cat([torch.arange(n - q, n) for n, q in zip(lengths, q_lens)]).to(torch.int32)
    seq = torch.cat([torch.full((q,), b) for b, q in enumerate(q_lens)]).to(torch.int32)
    scale = D ** -0.5
    out = torch.empty(T, H * D, dtype=DT[dtype], device="cuda")
    cu = torch.tensor([0, 75, 115, 116], dtype=torch.int32).cuda()
    ctx = SimpleNamespace(tok_pos=pos.cuda(), tok_seq=seq.cuda(), n_tokens=T, n_seqs=3, cu_q=cu,
                          kv_len=torch.tensor(lengths, dtype=torch.int32).cuda(), is_decode=False,
                          host_q_lens=q_lens, host_kv_lens=lengths, max_q_len=75, max_kv_len=301, extras={})
    ops.attention(qkv, out, KVLayerView(kp, vp, table, None), ctx, H, K, D, scale, window)
    q = qkv.double().cpu().view(T, H + 2 * K, D)[:, :H]
    t0 = 0
    for b, (n, ql) in enumerate(zip(lengths, q_lens)):
        want = ref_attention(q[t0:t0 + ql], ks[b].double().cpu(), vs[b].double().cpu(), pos[t0:t0 + ql], scale, window)
        close(out[t0:t0 + ql].view(ql, H, D), want, dtype, f"sequence {b}")
        t0 += ql


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key(dtype):
    """Among hundreds of keys one, far back and on another page, matches the query: the
    output must be its value.  A kernel that skips, misplaces or masks that key shows here."""
    from alpacca_b200 import ops
    from alpacca_b200.cache import KVLayerView
    from types import SimpleNamespace
    H, K, D, n = 4, 2, 64, 700
    table, kp, vp = make_paged([n], 16, K, D, DT[dtype], seed=3)
    kk = rnd(n, K, D, seed=1) * 0.1
    vv = rnd(n, K, D, seed=2)
    qkv = torch.zeros(1, (H + 2 * K) * D, device="cuda")
    far = {0: 5, 1: 64, 2: 383, 3: 699}      # page starts, page ends, the first and the very last key
    for h, s in far.items():
        direction = torch.zeros(D, device="cuda")
        direction[h * 7] = 1.0
        kk[s, h // 2] = direction * 30.0
        qkv[0, h * D:(h + 1) * D] = direction * 30.0
    fill_cache(table.cpu(), kp, vp, 0, kk, vv)
    qkv = qkv.to(DT[dtype])
    out = torch.empty(1, H * D, dtype=DT[dtype], device="cuda")
    ctx = SimpleNamespace(tok_pos=torch.tensor([n - 1], dtype=torch.int32).cuda(),
                          tok_seq=torch.zeros(1, dtype=torch.int32).cuda(), n_tokens=1, n_seqs=1,
                          cu_q=torch.tensor([0, 1], dtype=torch.int32).cuda(),
                          kv_len=torch.tensor([n], dtype=torch.int32).cuda(), is_decode=True,
                          host_q_lens=[1], host_kv_lens=[n], max_q_len=1, max_kv_len=n, extras={})
    ops.attention(qkv, out, KVLayerView(kp, vp, table, None), ctx, H, K, D, D ** -0.5, 0)
    for h, s in far.items():
        want = vp[table[0, s // 64].item(), h // 2, s % 64].float()
        got = out[0, h * D:(h + 1) * D].float()
        assert (got - want).abs().max().item() < 2e-2, f"head {h} did not find key {s}"
    # with a window the far keys are cut off, except the last one, which lies inside it
    ops.attention(qkv, out, KVLayerView(kp, vp, table, None), ctx, H, K, D, D ** -0.5, 100)
    want = vp[table[0, 699 // 64].item(), 1, 699 % 64].float()
    assert (out[0, 3 * D:].float() - want).abs().max().item() < 2e-2
    # the window's edge: position n-100 is the first key inside, n-101 the last one outside
    kk2 = kk.clone()
    kk2[600, 0] = kk[5, 0]       # head 0's matching key, now on the edge
    kk2[599, 1] = kk[383, 1]     # head 2's matching key, now just outside (its old place 383 is outside too)
    fill_cache(table.cpu(), kp, vp, 0, kk2, vv)
    ops.attention(qkv, out, KVLayerView(kp, vp, table, None), ctx, H, K, D, D ** -0.5, 100)
    edge = vp[table[0, 600 // 64].item(), 0, 600 % 64].float()
    assert (out[0, :D].float() - edge).abs().max().item() < 2e-2, "the key on the window's edge was not seen"
    outside = vp[table[0, 599 // 64].item(), 1, 599 % 64].float()
    assert (out[0, 2 * D:3 * D].float() - outside).abs().max().item() > 0.1, "a key outside the window was seen"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,F", [(1, 160), (9, 264), (70, 1000)])
def test_swiglu(dtype, T, F):
    from alpacca_b200 import ops
    gate, up = rnd(T, F, seed=1) * 3, rnd(T, F, seed=2)
    gu = torch.cat([gate.view(T, F // 8, 8), up.view(T, F // 8, 8)], dim=2).reshape(T, 2 * F).to(DT[dtype])
    g, u = gu.view(T, F // 8, 2, 8)[:, :, 0].reshape(T, F).double(), gu.view(T, F // 8, 2, 8)[:, :, 1].reshape(T, F).double()
    out = torch.empty(T, F, dtype=DT[dtype], device="cuda")
    ops.swiglu(gu, out)
    close(out, g / (1 + torch.exp(-g)) * u, dtype)


@pytest.mark.parametrize("M,N,K", [(1, 72, 200), (5, 1003, 120), (70, 264, 333), (130, 64, 64)])
def test_gemm_f32(M, N, K):
    from alpacca_b200 import ops
    a, w, bias = rnd(M, K, seed=1), rnd(N, K, seed=2), rnd(N, seed=3)
    out = torch.empty(M, N, device="cuda")
    ops.gemm_f32(a, w, out, bias=bias)
    close(out, a.double() @ w.double().T + bias.double(), "float32")
    # a row's result does not depend on the rows beside it
    out1 = torch.empty(1, N, device="cuda")
    ops.gemm_f32(a[M // 2:M // 2 + 1].contiguous(), w, out1, bias=bias)
    assert torch.equal(out1[0], out[M // 2])


@pytest.mark.parametrize("M,N,K", [(1, 72, 200), (3, 1003, 120), (8, 264, 328), (16, 520, 64), (70, 264, 336)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_linear_bf16(M, N, K, out_dtype):
    from alpacca_b200 import ops
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2)
    out = torch.empty(M, N, dtype=DT[out_dtype], device="cuda")
    ops.linear_bf16(a, w, out)
    want = a.double() @ w.double().T
    close(out, want, out_dtype if out_dtype == "bfloat16" else "float32", "linear_bf16")


def test_add_bias():
    from alpacca_b200 import ops
    y, b = rnd(7, 72, dtype=torch.bfloat16), rnd(72, seed=4)
    want = y.float() + b
    ops.add_bias(y, b)
    close(y, want, "bfloat16")


def decode_ctx(lengths):
    from types import SimpleNamespace
    B = len(lengths)
    return SimpleNamespace(
        tok_pos=torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda(),
        tok_seq=torch.arange(B, dtype=torch.int32).cuda(), n_tokens=B, n_seqs=B,
        cu_q=torch.arange(B + 1, dtype=torch.int32).cuda(), kv_len=torch.tensor(lengths, dtype=torch.int32).cuda(),
        is_decode=True, host_q_lens=[1] * B, host_kv_lens=list(lengths), max_q_len=1, max_kv_len=max(lengths),
        extras={})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,K,D", ATT_CASES + [(40, 2, 64)])
@pytest.mark.parametrize("window", [0, 130])
def test_attention_decode_batch(dtype, H, K, D, window):
    """One token per sequence, lengths from 1 to beyond a thousand keys (one to several chunks)."""
    from alpacca_b200 import ops
    from alpacca_b200.cache import KVLayerView
    lengths = [1, 64, 65, 300, 700, 1025]
    table, kp, vp = make_paged(lengths, 40, K, D, DT[dtype], seed=D + H)
    B = len(lengths)
    qkv = rnd(B, (H + 2 * K) * D, dtype=DT[dtype], seed=17)
    ks = [rnd(n, K, D, dtype=DT[dtype], seed=18 + b) for b, n in enumerate(lengths)]
    vs = [rnd(n, K, D, dtype=DT[dtype], seed=31 + b) for b, n in enumerate(lengths)]
    for b in range(B):
        fill_cache(table.cpu(), kp, vp, b, ks[b], vs[b])
    ctx = decode_ctx(lengths)
    out = torch.empty(B, H * D, dtype=DT[dtype], device="cuda")
    ops.attention(qkv, out, KVLayerView(kp, vp, table, None), ctx, H, K, D, D ** -0.5, window)
    q = qkv.double().cpu().view(B, H + 2 * K, D)[:, :H]
    for b, n in enumerate(lengths):
        want = ref_attention(q[b:b + 1], ks[b].double().cpu(), vs[b].double().cpu(), [n - 1], D ** -0.5, window)
        close(out[b].view(1, H, D), want, dtype, f"sequence of {n}")
    # a padded row (tok_seq -1) is skipped and leaves its output alone
    ctx.tok_seq[2] = -1
    out2 = torch.full_like(out, 7.0)
    ops.attention(qkv, out2, KVLayerView(kp, vp, table, None), ctx, H, K, D, D ** -0.5, window)
    assert torch.equal(out2[2], torch.full_like(out2[2], 7.0)) and torch.equal(out2[3], out[3])


@pytest.mark.parametrize("H,K,D", [(6, 2, 32), (8, 1, 64), (3, 3, 72)])
def test_attention_32bit_kernel_on_bfloat16(H, K, D):
    """The 32-bit kernel also serves bfloat16 tensors (head sizes the tensor-core kernel refuses)."""
    from alpacca_b200 import ops
    lengths = [5, 200]
    table, kp, vp = make_paged(lengths, 6, K, D, torch.bfloat16, seed=D)
    qkv = rnd(2, (H + 2 * K) * D, dtype=torch.bfloat16, seed=3)
    ks = [rnd(n, K, D, dtype=torch.bfloat16, seed=4 + b) for b, n in enumerate(lengths)]
    vs = [rnd(n, K, D, dtype=torch.bfloat16, seed=6 + b) for b, n in enumerate(lengths)]
    for b in range(2):
        fill_cache(table.cpu(), kp, vp, b, ks[b], vs[b])
    ctx = decode_ctx(lengths)
    out = torch.empty(2, H * D, dtype=torch.bfloat16, device="cuda")
    ops.attention_simt(qkv, out, kp, vp, table, ctx.tok_pos, ctx.tok_seq, 2, H, K, D, D ** -0.5, 0)
    q = qkv.double().cpu().view(2, H + 2 * K, D)[:, :H]
    for b, n in enumerate(lengths):
        want = ref_attention(q[b:b + 1], ks[b].double().cpu(), vs[b].double().cpu(), [n - 1], D ** -0.5)
        close(out[b].view(1, H, D), want, "bfloat16")


@pytest.mark.parametrize("M", [1, 5, 8, 13, 16, 27, 32])
@pytest.mark.parametrize("N,K", [(72, 200), (1003, 120), (2048, 2048), (264, 8200)])
def test_gemv_bf16(M, N, K):
    from alpacca_b200 import ops
    x, w, bias = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.1), rnd(N, seed=3)
    want = x.double() @ w.double().T + bias.double()
    for dt, tol in ((torch.float32, "float32"), (torch.bfloat16, "bfloat16")):
        out = torch.full((M, N), 9.0, dtype=dt, device="cuda")
        ops.gemv_bf16(x, w, out, bias=bias)
        close(out, want, tol, f"gemv {dt}")
    # fewer rows than the buffers hold: the rest is left alone
    if M > 1:
        out = torch.full((M, N), 9.0, dtype=torch.float32, device="cuda")
        ops.gemv_bf16(x, w, out, n_rows=M - 1)
        assert (out[M - 1] == 9.0).all()
        close(out[:M - 1], (x.double() @ w.double().T)[:M - 1], "float32")


@pytest.mark.parametrize("M,F,K", [(1, 160, 64), (7, 264, 120), (16, 1000, 328)])
def test_gemv_bf16_swiglu_epilogue(M, F, K):
    from alpacca_b200 import ops
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    gate, up = rnd(F, K, dtype=torch.bfloat16, seed=2, scale=0.3), rnd(F, K, dtype=torch.bfloat16, seed=3, scale=0.3)
    bg, bu = rnd(F, seed=4), rnd(F, seed=5)
    w = torch.cat([gate.view(F // 8, 8, K), up.view(F // 8, 8, K)], dim=1).reshape(2 * F, K).contiguous()
    bias = torch.cat([bg.view(F // 8, 8), bu.view(F // 8, 8)], dim=1).reshape(2 * F).contiguous()
    g = x.double() @ gate.double().T + bg.double()
    u = x.double() @ up.double().T + bu.double()
    out = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    ops.gemv_bf16(x, w, out, bias=bias, swiglu=True)
    close(out, g / (1 + torch.exp(-g)) * u, "bfloat16", "swiglu epilogue")


@pytest.mark.parametrize("M", [1, 5, 8, 13, 32])
@pytest.mark.parametrize("E,K,N2,slices", [(72, 200, 88, 1), (2048, 264, 1003, 1), (200, 8200, 72, 1),
                                           (4104, 128, 160, 1), (264, 4096, 520, 3)])
def test_gemv_bf16_norm_between_two_products(M, E, K, N2, slices):
    """The residual epilogue (add to the 32-bit residual, bf16(residual * norm weight), partial sums of
    squares) and the product after it that applies the owed division by the rms: together they are
    product, residual add, RMS norm (alpacca/tensor.py:163-173), product; also with the activation."""
    from alpacca_b200 import ops
    eps = 3e-4
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    w1, b1 = rnd(E, K, dtype=torch.bfloat16, seed=2, scale=0.1), rnd(E, seed=3)
    res0 = rnd(M, E, seed=4, scale=2.0)
    nw = 1.0 + rnd(E, seed=5, scale=0.3)
    w2, b2 = rnd(N2, E, dtype=torch.bfloat16, seed=6, scale=0.1), rnd(N2, seed=7)
    want_res = res0.double() + x.double() @ w1.double().T + b1.double()
    rms = torch.sqrt((want_res ** 2).mean(-1, keepdim=True) + eps)
    normed = want_res / rms * nw.double()
    want = normed @ w2.double().T + b2.double()

    res = res0.clone()
    xw = torch.full((M, E), 9.0, dtype=torch.bfloat16, device="cuda")
    _, ss = ops.gemv_bf16(x, w1, xw, bias=b1, residual=res, norm_weight=nw, slices=slices)
    close(res, want_res, "float32", "residual after the product")
    assert tuple(ss.shape) == (M, -(-E // 16))
    close(ss.sum(-1), (want_res ** 2).sum(-1), "float32", "sums of squares")
    close(xw, want_res * nw.double(), "bfloat16", "residual times the norm weight")
    owed = (ss, E, eps)
    for dt in (torch.float32, torch.bfloat16):
        out = torch.full((M, N2), 9.0, dtype=dt, device="cuda")
        ops.gemv_bf16(xw, w2, out, bias=b2, owed=owed)
        close(out, want, "bfloat16", f"product after the norm {dt}")
    if N2 % 16 == 0:
        F = N2 // 2
        g = want.view(M, F // 8, 2, 8)[:, :, 0].reshape(M, F)
        u = want.view(M, F // 8, 2, 8)[:, :, 1].reshape(M, F)
        out = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
        ops.gemv_bf16(xw, w2, out, bias=b2, swiglu=True, owed=owed)
        close(out, g / (1 + torch.exp(-g)) * u, "bfloat16", "activation after the norm")
    # fewer rows than the buffers hold: the rest of the residual is left alone
    if M > 1:
        res = res0.clone()
        ops.gemv_bf16(x, w1, xw, bias=b1, residual=res, norm_weight=nw, n_rows=M - 1)
        assert torch.equal(res[M - 1], res0[M - 1])
        close(res[:M - 1], want_res[:M - 1], "float32")


@pytest.mark.parametrize("M,N,K", [(3, 1003, 120), (8, 70, 64), (16, 2050, 264)])
def test_gemv_bf16_residual_epilogue_at_odd_widths(M, N, K):
    """The residual epilogue where the stream's width is no multiple of 4 (the tile of the residual is
    then read straight from memory, not staged) and the last slab is partial."""
    from alpacca_b200 import ops
    x, w, b = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.1), rnd(N, seed=3)
    res0, nw = rnd(M, N, seed=4, scale=2.0), 1.0 + rnd(N, seed=5, scale=0.3)
    want = res0.double() + x.double() @ w.double().T + b.double()
    res, xw = res0.clone(), torch.full((M, N), 9.0, dtype=torch.bfloat16, device="cuda")
    _, ss = ops.gemv_bf16(x, w, xw, bias=b, residual=res, norm_weight=nw)
    close(res, want, "float32", "residual")
    close(xw, want * nw.double(), "bfloat16", "residual times the norm weight")
    close(ss.sum(-1), (want ** 2).sum(-1), "float32", "sums of squares")


@pytest.mark.parametrize("M,N,K,swap,bn,slices", [
    (128, 256, 64, False, 256, 1), (300, 520, 328, False, 128, 1), (2048, 1024, 512, False, 256, 1),
    (8, 128, 128, True, 16, 1), (13, 1003, 200, True, 16, 1), (33, 520, 264, True, 64, 1),
    (64, 2048, 2048, True, 64, 4), (20, 264, 4096, True, 32, 3)])
def test_gemm_tc(M, N, K, swap, bn, slices):
    """The tcgen05 product in both orientations, with ragged edges, K slices and both output types."""
    from alpacca_b200 import ops
    x, w, bias = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.1), rnd(N, seed=3)
    want = x.double() @ w.double().T + bias.double()
    for dt, tol in ((torch.float32, "float32"), (torch.bfloat16, "bfloat16")):
        out = torch.full((M, N), 9.0, dtype=dt, device="cuda")
        ops.gemm_tc(x, w, out, bias=bias, swap=swap, bn=bn, slices=slices)
        close(out, want, tol, f"gemm_tc {dt}")
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("M,F,K,swap,bn", [(9, 160, 64, True, 16), (64, 264, 328, True, 64), (300, 1000, 200, False, 128),
                                           (128, 512, 256, False, 256)])
def test_gemm_tc_swiglu_epilogue(M, F, K, swap, bn):
    from alpacca_b200 import ops
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    gate, up = rnd(F, K, dtype=torch.bfloat16, seed=2, scale=0.3), rnd(F, K, dtype=torch.bfloat16, seed=3, scale=0.3)
    bg, bu = rnd(F, seed=4), rnd(F, seed=5)
    w = torch.cat([gate.view(F // 8, 8, K), up.view(F // 8, 8, K)], dim=1).reshape(2 * F, K).contiguous()
    bias = torch.cat([bg.view(F // 8, 8), bu.view(F // 8, 8)], dim=1).reshape(2 * F).contiguous()
    g = x.double() @ gate.double().T + bg.double()
    u = x.double() @ up.double().T + bu.double()
    out = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc(x, w, out, bias=bias, swiglu=True, swap=swap, bn=bn, slices=1)
    close(out, g / (1 + torch.exp(-g)) * u, "bfloat16", "tcgen05 swiglu epilogue")
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("H,K,D", [(4, 4, 64), (8, 2, 64), (32, 8, 64), (16, 1, 64), (6, 6, 64), (6, 2, 64), (10, 2, 64),
                                   (4, 4, 128), (8, 2, 128), (16, 1, 128), (12, 2, 128), (7, 1, 128)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("growing", [False, True])
def test_attention_prefill_tcgen05(H, K, D, window, growing):
    """The tcgen05 prefill kernel (head sizes 64 and 128): whole prompts, a chunk on cached tokens,
    several sequences in one launch; against the float64 reference and against the mma.sync kernel.
    `growing`: the keys get longer with their position, so that the rows' maxima keep rising by large
    steps and the kernel has to move its references and rescale its output again and again."""
    from alpacca_b200 import ops
    from alpacca_b200.cache import KVLayerView
    from types import SimpleNamespace
    lengths, q_lens = [300, 150, 513], [300, 100, 130]
    table, kp, vp = make_paged(lengths, 20, K, D, torch.bfloat16, seed=H)
    T = sum(q_lens)
    qkv = rnd(T, (H + 2 * K) * D, dtype=torch.bfloat16, seed=7)
    ks = [rnd(n, K, D, dtype=torch.bfloat16, seed=8 + b) for b, n in enumerate(lengths)]
    vs = [rnd(n, K, D, dtype=torch.bfloat16, seed=11 + b) for b, n in enumerate(lengths)]
    if growing:
        ks = [(k.float() * (1.0 + torch.arange(k.shape[0], device=k.device).view(-1, 1, 1) / 16.0)).to(torch.bfloat16)
              for k in ks]
    for b in range(3):
        fill_cache(table.cpu(), kp, vp, b, ks[b], vs[b])
    pos = torch.cat([torch.arange(n - q, n) for n, q in zip(lengths, q_lens)]).to(torch.int32)
    seq = torch.cat([torch.full((q,), b) for b, q in enumerate(q_lens)]).to(torch.int32)
    cu = torch.tensor([0, 300, 400, 530], dtype=torch.int32).cuda()

    def run(use_tc):
        ctx = SimpleNamespace(tok_pos=pos.cuda(), tok_seq=seq.cuda(), n_tokens=T, n_seqs=3, cu_q=cu,
                              kv_len=torch.tensor(lengths, dtype=torch.int32).cuda(), is_decode=False,
                              host_q_lens=q_lens, host_kv_lens=lengths, max_q_len=300, max_kv_len=513, extras={})
        out = torch.zeros(T, H * D, dtype=torch.bfloat16, device="cuda")
        old = ops.USE_TCGEN05_ATTENTION
        ops.USE_TCGEN05_ATTENTION = use_tc
        try:
            ops.attention(qkv, out, KVLayerView(kp, vp, table, None), ctx, H, K, D, D ** -0.5, window)
        finally:
            ops.USE_TCGEN05_ATTENTION = old
        return out
    got, other = run(True), run(False)
    assert ops.attention_tc_status() == 0
    q = qkv.double().cpu().view(T, H + 2 * K, D)[:, :H]
    t0 = 0
    for b, (n, ql) in enumerate(zip(lengths, q_lens)):
        want = ref_attention(q[t0:t0 + ql], ks[b].double().cpu(), vs[b].double().cpu(), pos[t0:t0 + ql], D ** -0.5, window)
        close(got[t0:t0 + ql].view(ql, H, D), want, "bfloat16", f"tcgen05, sequence {b}")
        close(other[t0:t0 + ql].view(ql, H, D), want, "bfloat16", f"mma.sync, sequence {b}")
        t0 += ql


@pytest.mark.parametrize("H,K,D,n_rot,pairing", [(4, 4, 16, 16, 0), (6, 2, 32, 32, 1), (10, 5, 48, 32, 1),
                                                 (32, 8, 64, 64, 1), (4, 2, 128, 64, 0), (40, 2, 64, 0, 0)])
@pytest.mark.parametrize("window", [0, 130])
@pytest.mark.parametrize("write_cache", [True, False])
def test_rope_attention_fused_decode(H, K, D, n_rot, pairing, window, write_cache):
    """Rotation, append and attention of a decode step in one kernel against the two kernels one
    after the other: the same outputs and the same cache, bit for bit; one to several chunks."""
    from alpacca_b200 import ops
    from alpacca_b200.cache import KVLayerView
    lengths = [1, 64, 65, 300, 769, 1025, 1600]
    B = len(lengths)
    qkv0 = rnd(B, (H + 2 * K) * D, dtype=torch.bfloat16, seed=17)
    ang = rnd(1700, max(n_rot // 2, 1), seed=5, scale=3.0)
    rot = (torch.cos(ang).contiguous(), torch.sin(ang).contiguous(), n_rot, pairing) if n_rot else None
    results = []
    for fused in (False, True):
        table, kp, vp = make_paged(lengths, 70, K, D, torch.bfloat16, seed=D + H)
        for b, n in enumerate(lengths):
            # with write_cache off the step's own row is in the cache already (another layer's)
            fill_cache(table.cpu(), kp, vp, b, rnd(n, K, D, dtype=torch.bfloat16, seed=18 + b),
                       rnd(n, K, D, dtype=torch.bfloat16, seed=31 + b))
        ctx = decode_ctx(lengths)
        ctx.tok_seq[2] = -1                      # a padding row: no output, nothing appended
        qkv = qkv0.clone()
        out = torch.full((B, H * D), 7.0, dtype=torch.bfloat16, device="cuda")
        ops.FUSE_ROPE_DECODE = fused
        try:
            ops.rope_attention(qkv, out, KVLayerView(kp, vp, table, None), ctx, H, K, D, D ** -0.5, window, rot,
                               write_cache=write_cache)
        finally:
            ops.FUSE_ROPE_DECODE = True
        results.append((out, kp, vp))
    (o1, k1, v1), (o2, k2, v2) = results
    assert torch.equal(o1, o2), f"outputs differ by {(o1.float() - o2.float()).abs().max().item()}"
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert (o1[3].float().abs() > 0).any() and torch.equal(o1[2], torch.full_like(o1[2], 7.0))


@pytest.mark.parametrize("H,K,D,B", [(8, 4, 64, 50), (8, 4, 64, 90), (4, 4, 128, 80), (2, 2, 256, 160), (24, 1, 64, 200)])
def test_attention_decode_many_sequences(H, K, D, B):
    """More (sequence, head) pairs than processors: the smaller CTAs, several rounds each; lengths
    from one key to several rounds' worth, with a window on top."""
    from alpacca_b200 import ops
    from alpacca_b200.cache import KVLayerView
    lengths = [1 + (37 * b * b + 11 * b) % 700 for b in range(B)]
    table, kp, vp = make_paged(lengths, sum(-(-n // 64) for n in lengths) + 3, K, D, torch.bfloat16, seed=B)
    qkv = rnd(B, (H + 2 * K) * D, dtype=torch.bfloat16, seed=17)
    check = sorted(set([0, 1, B // 2, B - 1, max(range(B), key=lambda b: lengths[b])]))
    ks, vs = {}, {}
    for b, n in enumerate(lengths):
        kk, vv = rnd(n, K, D, dtype=torch.bfloat16, seed=18 + b), rnd(n, K, D, dtype=torch.bfloat16, seed=931 + b)
        fill_cache(table.cpu(), kp, vp, b, kk, vv)
        if b in check:
            ks[b], vs[b] = kk, vv
    ctx = decode_ctx(lengths)
    q = qkv.double().cpu().view(B, H + 2 * K, D)[:, :H]
    for window in (0, 100):
        out = torch.empty(B, H * D, dtype=torch.bfloat16, device="cuda")
        ops.attention(qkv, out, KVLayerView(kp, vp, table, None), ctx, H, K, D, D ** -0.5, window)
        for b in check:
            want = ref_attention(q[b:b + 1], ks[b].double().cpu(), vs[b].double().cpu(), [lengths[b] - 1], D ** -0.5, window)
            close(out[b].view(1, H, D), want, "bfloat16", f"sequence {b} of {lengths[b]}, window {window}")


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,N,K", [(2500, 2100, 328), (4000, 3000, 200), (130, 300, 4104), (256, 256, 64), (20000, 700, 520)])
def test_gemm_tc_persistent(M, N, K, pair):
    """The persistent form of the tcgen05 product: more tiles than processors (a CTA walks several,
    both accumulator buffers in turn), ragged edges in every direction, both output types; `pair`: on
    pairs of processors (tiles of 256 x 256 by `tcgen05.mma.cta_group::2`)."""
    from alpacca_b200 import ops
    x, w, bias = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.1), rnd(N, seed=3)
    want = x.double() @ w.double().T + bias.double()
    for dt, tol in ((torch.float32, "float32"), (torch.bfloat16, "bfloat16")):
        out = torch.full((M, N), 9.0, dtype=dt, device="cuda")
        ops.gemm_tc(x, w, out, bias=bias, swap=False, bn=256, slices=1, pair=pair)
        close(out, want, tol, f"persistent gemm_tc {dt}")
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,F,K", [(3000, 1304, 264), (1024, 512, 2048)])
def test_gemm_tc_persistent_swiglu(M, F, K, pair):
    from alpacca_b200 import ops
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    gate, up = rnd(F, K, dtype=torch.bfloat16, seed=2, scale=K ** -0.5), rnd(F, K, dtype=torch.bfloat16, seed=3, scale=K ** -0.5)
    bg, bu = rnd(F, seed=4), rnd(F, seed=5)
    w = torch.cat([gate.view(F // 8, 8, K), up.view(F // 8, 8, K)], dim=1).reshape(2 * F, K).contiguous()
    bias = torch.cat([bg.view(F // 8, 8), bu.view(F // 8, 8)], dim=1).reshape(2 * F).contiguous()
    g = x.double() @ gate.double().T + bg.double()
    u = x.double() @ up.double().T + bu.double()
    out = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc(x, w, out, bias=bias, swiglu=True, swap=False, pair=pair)
    close(out, g / (1 + torch.exp(-g)) * u, "bfloat16", "persistent swiglu epilogue")
    assert ops.gemm_tc_status() == 0
