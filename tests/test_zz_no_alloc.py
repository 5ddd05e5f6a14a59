"""The decode-attention entry point that allocates nothing, called the way an outside caller
would: through its exported C symbol, with raw pointers.

Such a caller cannot allocate device memory when it calls (its memory was handed out at start-up,
or it sits in a loop that must not synchronise the device), so the scratch memory of the split over
key chunks lives inside the library.  This test checks that the entry point gives what the package's
own entry point gives when that one is handed scratch tensors, twice in a row (the second call finds
the scratch as the first left it), that both agree with a float64 restatement of the attention on the
same inputs (with and without a window, with a row of the batch that holds no sequence), that a call
leaves the device's free memory as it found it, and that it refuses problems beyond either of its
stated limits.

The file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(lengths, H, K, D, seed):
    g = torch.Generator().manual_seed(seed)
    B = len(lengths)
    n_pages = sum(-(-n // 64) for n in lengths) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // 64) for n in lengths)
    table = torch.zeros(B, width, dtype=torch.int32)
    for b, n in enumerate(lengths):
        for i in range(-(-n // 64)):
            table[b, i] = perm.pop()
    k = (torch.randn(n_pages, K, 64, D, generator=g)).to(torch.bfloat16).cuda()
    v = (torch.randn(n_pages, K, 64, D, generator=g)).to(torch.bfloat16).cuda()
    qkv = torch.randn(B, (H + 2 * K) * D, generator=g).to(torch.bfloat16).cuda()
    return qkv, k, v, table.cuda(), torch.arange(B, dtype=torch.int32).cuda(), \
        torch.tensor(lengths, dtype=torch.int32).cuda()


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _plain_attention(qkv, k, v, table, seq, lens, H, K, D, window):
    """softmax(q . k / sqrt(D)) v over each sequence's keys (the last `window` of them), float64;
    a row whose `seq` is -1 holds no sequence and is left at zero."""
    qkv, k, v = qkv.double().cpu(), k.double().cpu(), v.double().cpu()
    table, seq, lens = table.cpu(), seq.tolist(), lens.tolist()
    out = torch.zeros(len(seq), H * D, dtype=torch.float64)
    G = H // K
    for row, b in enumerate(seq):
        if b < 0:
            continue
        n = lens[b]
        pages = table[b, :-(-n // 64)].long()
        lo = max(0, n - window) if window else 0
        for h in range(H):
            keys = k[pages, h // G].reshape(-1, D)[lo:n]
            vals = v[pages, h // G].reshape(-1, D)[lo:n]
            p = torch.softmax(keys @ qkv[row, h * D:(h + 1) * D] * D ** -0.5, dim=0)
            out[row, h * D:(h + 1) * D] = p @ vals
    return out


def test_no_alloc_entry_point_matches_the_package_s_own():
    from alpacca_b200.ops import build
    lib = build.load("attention_mma")
    lib.ab_attention_decode_bf16_noalloc_error.restype = ctypes.c_char_p
    H, K, D = 8, 2, 64
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ppc = 2          # pages per chunk: more than 8 chunks, which are merged through the scratch memory
    cases = (([1500, 70, 2048, 1025], 0, None), ([900, 2047, 33, 1300], 0, None),
             ([1100, 2040, 64, 700], 300, 2))        # the last: a window of 300 keys, and row 2 holds no sequence
    for call, (lengths, window, empty_row) in enumerate(cases):   # several chunks each
        qkv, k, v, table, seq, lens = _setup(lengths, H, K, D, seed=call)
        if empty_row is not None:
            seq[empty_row] = -1
        B, W = table.shape
        n_chunks = -(-W // ppc)
        assert n_chunks > 8, "the case must need the scratch memory"
        # the package's entry point, with scratch tensors of its caller
        want = torch.zeros(B, H * D, dtype=torch.bfloat16, device="cuda")
        part_o = torch.empty(B * H * n_chunks * D, dtype=torch.float32, device="cuda")
        part_ml = torch.empty(B * H * n_chunks * 2, dtype=torch.float32, device="cuda")
        arrivals = torch.zeros(B * K, dtype=torch.int32, device="cuda")
        rc = lib.ab_attention_decode_bf16(_p(qkv), qkv.shape[1], _p(want), _p(part_o), _p(part_ml), _p(arrivals),
                                          _p(k), _p(v), _p(table), W, _p(seq), _p(lens), B, H, K, D,
                                          ctypes.c_float(D ** -0.5), window, ppc, n_chunks, 0, stream)
        assert rc == 0
        # what the attention is, restated in float64 on the same inputs
        plain = _plain_attention(qkv, k, v, table, seq, lens, H, K, D, window).cuda()
        assert (want.double() - plain).abs().max().item() <= 1.6e-2
        # few chunks, merged inside a cluster without scratch: the same result by another route
        few = torch.zeros(B, H * D, dtype=torch.bfloat16, device="cuda")
        rc = lib.ab_attention_decode_bf16(_p(qkv), qkv.shape[1], _p(few), None, None, None, _p(k), _p(v), _p(table),
                                          W, _p(seq), _p(lens), B, H, K, D, ctypes.c_float(D ** -0.5), window, 8,
                                          -(-W // 8), 0, stream)
        assert rc == 0
        assert (few.float() - want.float()).abs().max().item() <= 1.6e-2
        # the entry point that allocates nothing: inputs and output only
        got = torch.zeros(B, H * D, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        # the device's free memory, as the driver counts it, whoever allocates (the first call of a
        # process may still load the kernel's code, so the comparison starts with the second)
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.ab_attention_decode_bf16_noalloc(_p(qkv), qkv.shape[1], _p(got), _p(k), _p(v), _p(table), W,
                                                  _p(seq), _p(lens), B, H, K, D, ctypes.c_float(D ** -0.5), window,
                                                  ppc, n_chunks, stream)
        assert rc == 0, lib.ab_attention_decode_bf16_noalloc_error()
        torch.cuda.synchronize()
        if call:
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        assert (got.double() - plain).abs().max().item() <= 1.6e-2
        if empty_row is not None:
            assert got[empty_row].float().abs().max().item() == 0.0, "a row without a sequence was written"
        # the same kernel with the same inputs: the tolerance of the kernel tests (bfloat16 outputs of order 1)
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 1.6e-2, f"call {call}: max difference {err}"
        assert got.float().abs().max().item() > 0.01


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from alpacca_b200.ops import build
    lib = build.load("attention_mma")
    lib.ab_attention_decode_bf16_noalloc_error.restype = ctypes.c_char_p
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    # 64 tokens x 64 heads x 8 chunks x 256 > 2^20 floats of partial outputs
    rc = lib.ab_attention_decode_bf16_noalloc(_p(dummy), 0, _p(dummy), _p(dummy), _p(dummy), _p(dummy), 128,
                                              _p(dummy), _p(dummy), 64, 64, 8, 256, ctypes.c_float(1.0), 0, 16, 8,
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 2
    assert b"too large" in lib.ab_attention_decode_bf16_noalloc_error()
    # the other limit alone: 8,193 tokens x 8 KV heads = 65,544 counters > 2^16, while the partial
    # outputs (8,193 x 8 heads x 1 chunk x 8) stay below theirs
    rc = lib.ab_attention_decode_bf16_noalloc(_p(dummy), 0, _p(dummy), _p(dummy), _p(dummy), _p(dummy), 1,
                                              _p(dummy), _p(dummy), 8193, 8, 8, 8, ctypes.c_float(1.0), 0, 1, 1,
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 2
    msg = lib.ab_attention_decode_bf16_noalloc_error()
    assert b"65544 (limit 65536)" in msg and b"524352 (limit 1048576)" in msg
