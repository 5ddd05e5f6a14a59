"""The streamed decode attention (csrc/attention_stream.cu) alone: against a float64 restatement of
the attention at sizes other than the engine's, every way of cutting a sequence into chunks and of
merging them, and against the other decode kernel for the rotation and the append to the cache."""
import pytest
import torch

from test_gpu_kernels import close, decode_ctx, fill_cache, make_paged, ref_attention, rnd

pytestmark = pytest.mark.gpu

# (heads, KV heads, head size): groups of 1, 3, 4, 8 and 12 (two tiles of heads) query heads per KV head
CASES = [(4, 4, 64), (8, 1, 64), (32, 8, 64), (12, 1, 64), (4, 2, 128), (3, 1, 128), (16, 16, 128)]
# pages per CTA, merge, depth of the ring: one chunk; up to 8 chunks in a cluster; many chunks through memory
CUTS = [(32, "memory", 1), (32, "memory", 2), (32, "memory", 0), (4, "cluster", 1), (5, "memory", 0),
        (1, "memory", 1), (2, "memory", 2)]


@pytest.mark.parametrize("ppc,merge,ring", CUTS)
@pytest.mark.parametrize("window", [0, 130])
@pytest.mark.parametrize("H,K,D", CASES)
def test_against_a_plain_restatement(H, K, D, window, ppc, merge, ring):
    """Lengths from one key to 25 pages, page edges among them; the keys are in the cache already."""
    from alpacca_b200 import ops
    from alpacca_b200.cache import KVLayerView
    lengths = [1, 64, 65, 300, 700, 1025, 1600, 127, 128]
    table, kp, vp = make_paged(lengths, 96, K, D, torch.bfloat16, seed=D + H)
    B = len(lengths)
    qkv = rnd(B, (H + 2 * K) * D, dtype=torch.bfloat16, seed=17)
    ks = [rnd(n, K, D, dtype=torch.bfloat16, seed=18 + b) for b, n in enumerate(lengths)]
    vs = [rnd(n, K, D, dtype=torch.bfloat16, seed=31 + b) for b, n in enumerate(lengths)]
    # pages that no sequence owns hold large values: reading one would show
    kp.fill_(50.0)
    vp.fill_(-50.0)
    for b in range(B):
        fill_cache(table.cpu(), kp, vp, b, ks[b], vs[b])
    ctx = decode_ctx(lengths)
    if ring != 1:
        # the rows' CTAs start in another order (longest sequence first): the same results
        ctx.row_order = torch.tensor(sorted(range(B), key=lambda b: -lengths[b]), dtype=torch.int32).cuda()
    out = torch.full((B, H * D), 7.0, dtype=torch.bfloat16, device="cuda")
    view = KVLayerView(kp, vp, table, None)
    ops.attention_stream(qkv, out, view, ctx, H, K, D, D ** -0.5, window, pages_per_cta=ppc, merge=merge, ring=ring)
    q = qkv.double().cpu().view(B, H + 2 * K, D)[:, :H]
    for b, n in enumerate(lengths):
        want = ref_attention(q[b:b + 1], ks[b].double().cpu(), vs[b].double().cpu(), [n - 1], D ** -0.5, window)
        close(out[b].view(1, H, D), want, "bfloat16", f"sequence of {n}")
    # a row without a sequence is skipped and leaves its output alone; the others are as before
    ctx.tok_seq[2] = -1
    out2 = torch.full_like(out, 7.0)
    ops.attention_stream(qkv, out2, view, ctx, H, K, D, D ** -0.5, window, pages_per_cta=ppc, merge=merge, ring=ring)
    assert torch.equal(out2[2], torch.full_like(out2[2], 7.0)) and torch.equal(out2[3], out[3])
    assert torch.equal(out2[6], out[6]), "the same inputs gave other sums: the merge order is not fixed"
    assert ops.attention_stream_status() == 0


def test_one_far_key_among_thousands():
    """One key far back that matches the query stands out against thousands that do not, in a CTA of its
    own chunk; dropping a page or a chunk would lose it."""
    from alpacca_b200 import ops
    from alpacca_b200.cache import KVLayerView
    H, K, D = 8, 2, 64
    n = 3000
    for far in (0, 63, 64, 1500, 2943, n - 1):
        table, kp, vp = make_paged([n], 50, K, D, torch.bfloat16, seed=far)
        kk = rnd(n, K, D, dtype=torch.bfloat16, seed=3, scale=0.05)
        vv = rnd(n, K, D, dtype=torch.bfloat16, seed=4, scale=0.05)
        qkv = rnd(1, (H + 2 * K) * D, dtype=torch.bfloat16, seed=5)
        q = qkv.view(1, H + 2 * K, D)
        for kh in range(K):
            kk[far, kh] = (q[0, kh * (H // K)].float() * 4.0).to(torch.bfloat16)     # score of about 4 * |q|^2 / 8
            vv[far, kh] = 3.0
        fill_cache(table.cpu(), kp, vp, 0, kk, vv)
        ctx = decode_ctx([n])
        for ppc, merge in ((3, "memory"), (6, "cluster"), (64, "memory")):
            out = torch.zeros(1, H * D, dtype=torch.bfloat16, device="cuda")
            ops.attention_stream(qkv, out, KVLayerView(kp, vp, table, None), ctx, H, K, D, D ** -0.5, 0,
                                 pages_per_cta=ppc, merge=merge)
            want = ref_attention(qkv.double().cpu().view(1, H + 2 * K, D)[:, :H], kk.double().cpu(),
                                 vv.double().cpu(), [n - 1], D ** -0.5, 0)
            assert want.view(H, D)[0].mean().item() > 2.5, "the test's far key must carry the result"
            close(out.view(1, H, D), want, "bfloat16", f"far key at {far}, {ppc} pages per CTA")


@pytest.mark.parametrize("H,K,D,n_rot,pairing", [(32, 8, 64, 64, 1), (4, 2, 128, 64, 0), (40, 2, 64, 0, 0),
                                                 (8, 8, 128, 128, 1), (6, 2, 64, 32, 0)])
@pytest.mark.parametrize("window", [0, 130])
@pytest.mark.parametrize("write_cache", [True, False])
def test_rotation_and_append_inside_the_kernel(H, K, D, n_rot, pairing, window, write_cache):
    """Rotation of q and k, the append of k and v and the attention in this kernel against the other
    decode kernel: the same cache bit for bit (the rotation is the same arithmetic), the same outputs
    within rounding (the keys are added in another order)."""
    from alpacca_b200 import ops
    from alpacca_b200.cache import KVLayerView
    lengths = [1, 64, 65, 300, 769, 1025, 1600]
    B = len(lengths)
    qkv0 = rnd(B, (H + 2 * K) * D, dtype=torch.bfloat16, seed=17)
    ang = rnd(1700, max(n_rot // 2, 1), seed=5, scale=3.0)
    rot = (torch.cos(ang).contiguous(), torch.sin(ang).contiguous(), n_rot, pairing) if n_rot else None
    results = []
    for streamed in (False, True):
        table, kp, vp = make_paged(lengths, 70, K, D, torch.bfloat16, seed=D + H)
        for b, n in enumerate(lengths):
            fill_cache(table.cpu(), kp, vp, b, rnd(n, K, D, dtype=torch.bfloat16, seed=18 + b),
                       rnd(n, K, D, dtype=torch.bfloat16, seed=31 + b))
        ctx = decode_ctx(lengths)
        ctx.tok_seq[2] = -1                      # a row without a sequence: no output, nothing appended
        qkv = qkv0.clone()
        out = torch.full((B, H * D), 7.0, dtype=torch.bfloat16, device="cuda")
        view = KVLayerView(kp, vp, table, None)
        if streamed:
            ops.attention_stream(qkv, out, view, ctx, H, K, D, D ** -0.5, window, rot, fuse=2 if write_cache else 1,
                                 pages_per_cta=6, merge="memory")
        else:
            ops._attention_decode_mma(qkv, out, view, ctx, H, K, D, D ** -0.5, window, rot, 2 if write_cache else 1)
        results.append((out, kp, vp))
    (o1, k1, v1), (o2, k2, v2) = results
    assert torch.equal(k1, k2) and torch.equal(v1, v2), "the two kernels left different caches"
    close(o2, o1.double(), "bfloat16", "streamed against the other decode kernel")
    assert (o2[3].float().abs() > 0).any() and torch.equal(o2[2], torch.full_like(o2[2], 7.0))
    assert ops.attention_stream_status() == 0


def test_sizes_it_does_not_take_are_refused():
    from alpacca_b200 import ops
    from alpacca_b200.cache import KVLayerView
    H, K, D = 4, 2, 48
    table, kp, vp = make_paged([10], 2, K, D, torch.bfloat16)
    qkv = rnd(1, (H + 2 * K) * D, dtype=torch.bfloat16)
    out = torch.zeros(1, H * D, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="head size 48"):
        ops.attention_stream(qkv, out, KVLayerView(kp, vp, table, None), decode_ctx([10]), H, K, D, 1.0)
