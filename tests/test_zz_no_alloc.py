"""The decode-attention entry point that allocates nothing, called the way an outside caller
would: through its exported C symbol, with raw pointers.

Such a caller cannot allocate device memory when it calls (its memory was handed out at start-up,
or it sits in a loop that must not synchronise the device), so the scratch memory of the split over
key chunks lives inside the library.  This test checks that the entry point gives what the package's
own entry point gives when that one is handed scratch tensors, twice in a row (the second call finds
the scratch as the first left it), and that it refuses problems beyond its stated limit.

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


def test_no_alloc_entry_point_matches_the_package_s_own():
    from alpacca_b200.ops import build
    lib = build.load("attention_mma")
    lib.ab_attention_decode_bf16_noalloc_error.restype = ctypes.c_char_p
    H, K, D = 8, 2, 64
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ppc = 2          # pages per chunk: more than 8 chunks, which are merged through the scratch memory
    for call, lengths in enumerate(([1500, 70, 2048, 1025], [900, 2047, 33, 1300])):   # several chunks each
        qkv, k, v, table, seq, lens = _setup(lengths, H, K, D, seed=call)
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
                                          ctypes.c_float(D ** -0.5), 0, ppc, n_chunks, 0, stream)
        assert rc == 0
        # few chunks, merged inside a cluster without scratch: the same result by another route
        few = torch.zeros(B, H * D, dtype=torch.bfloat16, device="cuda")
        rc = lib.ab_attention_decode_bf16(_p(qkv), qkv.shape[1], _p(few), None, None, None, _p(k), _p(v), _p(table),
                                          W, _p(seq), _p(lens), B, H, K, D, ctypes.c_float(D ** -0.5), 0, 8,
                                          -(-W // 8), 0, stream)
        assert rc == 0
        assert (few.float() - want.float()).abs().max().item() <= 1.6e-2
        # the entry point that allocates nothing: inputs and output only
        got = torch.zeros(B, H * D, dtype=torch.bfloat16, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = lib.ab_attention_decode_bf16_noalloc(_p(qkv), qkv.shape[1], _p(got), _p(k), _p(v), _p(table), W,
                                                  _p(seq), _p(lens), B, H, K, D, ctypes.c_float(D ** -0.5), 0, ppc,
                                                  n_chunks, stream)
        assert rc == 0, lib.ab_attention_decode_bf16_noalloc_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
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
