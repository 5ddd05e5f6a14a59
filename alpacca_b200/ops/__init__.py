"""Python side of the CUDA kernels: argument checks and the ctypes calls.

Every function here runs a hand-written sm_100a kernel from `csrc/` on the
current CUDA stream.  There is no CPU implementation behind them: tensors that
are not on a CUDA device are refused, and a library that cannot be built or
loaded raises.  Shapes, dtypes, strides and index ranges that a kernel relies
on are checked here, on the host, before the launch, since a kernel given a
bad pointer or size would fault the device rather than raise.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import build

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


# The library products of this package (`torch.mm` on bfloat16 operands) add in float32 throughout: the
# library may not reduce partial sums of a split inner dimension in bfloat16 (measured on a B200 at the 1B
# sizes: the same step times and the same results either way; the setting makes it a rule).
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


def _lib(name):
    return build.load(name)


# torch's current stream of the current device as a raw handle.  The direct bindings cost a
# fraction of a microsecond; torch.cuda.current_stream() builds a Stream object each time
# (15 us, and a prefill step asks a hundred times).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _need(cond, msg):
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("alpacca_b200 kernels run on CUDA tensors only (there is no CPU path); "
                              f"got a tensor on {t.device}")


launches = 0     # kernels of this package launched so far (the benchmark reports the count)
_timeline = None  # while `timers()` is active: [(operation, event recorded after its launch), ...]


class Timers:
    """Device time per kind of operation, for steps that are issued one launch after the other (not for
    graph replays).  An event is recorded after every launch of this package (and after the library
    products it calls); an operation's time is the time from the event before it to its own, so what
    the device idles between two launches counts for the later one.

        with ops.timers() as t:
            engine.step(entries)
        print(t.table())
    """

    def __init__(self):
        self.marks = []

    def __enter__(self):
        global _timeline
        if _timeline is not None:
            raise KernelError("ops.timers() is already active")
        torch.cuda.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        self.marks = [("start", start)]
        _timeline = self.marks
        return self

    def __exit__(self, *exc):
        global _timeline
        _timeline = None
        torch.cuda.synchronize()
        return False

    def totals(self) -> dict:
        """{operation: (launches, microseconds)} in the order of first appearance."""
        out: dict = {}
        for (_, before), (what, after) in zip(self.marks, self.marks[1:]):
            n, us = out.get(what, (0, 0.0))
            out[what] = (n + 1, us + before.elapsed_time(after) * 1e3)
        return out

    def table(self) -> str:
        tot = self.totals()
        whole = sum(us for _, us in tot.values()) or 1.0
        lines = [f"{'operation':<24} {'launches':>8} {'us':>10} {'share':>7}"]
        for what, (n, us) in sorted(tot.items(), key=lambda kv: -kv[1][1]):
            lines.append(f"{what:<24} {n:>8} {us:>10.1f} {100 * us / whole:>6.1f}%")
        lines.append(f"{'total':<24} {sum(n for n, _ in tot.values()):>8} {whole:>10.1f}")
        return "\n".join(lines)


def timers() -> Timers:
    return Timers()


def timing() -> bool:
    """Whether `timers()` is active: every launch is followed by an event then, so nothing may be captured
    into a graph or replayed from one (a replay is opaque to the events)."""
    return _timeline is not None


def _mark(what):
    if _timeline is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        _timeline.append((what, ev))


def _check(rc, what):
    global launches
    launches += 1
    _mark(what)
    if rc != 0:
        if rc >= 1000:
            raise KernelError(f"{what}: CUDA error {rc - 1000} at launch")
        raise KernelError(f"{what}: the kernel refused its arguments (code {rc})")


def _dt(t):
    code = _DT.get(t.dtype)
    if code is None:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32 or bfloat16)")
    return code


def _i32(t, n=None, name="index tensor"):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    if n is not None and t.numel() < n:
        raise KernelError(f"{name} holds {t.numel()} entries, {n} needed")


# ---------------------------------------------------------------------------

def embed_rows(table, tokens, out):
    """out[i,:] = table[tokens[i],:] as float32.  table [V,E] f32/bf16, tokens int32 [n], out f32 [n,E]."""
    _cuda(table, tokens, out)
    n = tokens.numel()
    _i32(tokens, name="tokens")
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be contiguous [V,E]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape[-1] == table.shape[1]
          and out.numel() >= n * table.shape[1], "embed_rows: out must be float32 [n,E]")
    _check(_lib("elementwise").ab_embed_rows(_p(table), _dt(table), _p(tokens), _p(out), n,
                                             table.shape[1], table.shape[0], _stream()), "embed_rows")
    return out


def add_rmsnorm(residual, delta, weight, eps, out, rows=None, n_rows=None):
    """Fused residual add and RMSNorm.

    residual f32 [T,E] (updated in place with `delta` when `rows` is None),
    delta [T,E] of the activation dtype or None, weight f32 [E], out [n,E] of
    the activation dtype or None (add only).  `rows` (int32 [n]) picks the
    source rows and leaves the residual untouched.
    """
    _cuda(residual, delta, weight, out, rows)
    E = residual.shape[-1]
    T = residual.numel() // E
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "residual must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.numel() == E and weight.is_contiguous(),
          "norm weight must be float32 [E]")
    if delta is not None:
        _need(delta.is_contiguous() and delta.numel() == residual.numel(), "delta must match the residual")
    if rows is not None:
        n = rows.numel() if n_rows is None else n_rows
        _i32(rows, n, "rows")
    else:
        n = T if n_rows is None else n_rows
        _need(n <= T, "add_rmsnorm: more rows than the residual has")
    act = out if out is not None else delta
    _need(act is not None, "add_rmsnorm needs delta or out")
    if out is not None:
        _need(out.is_contiguous() and out.numel() >= n * E, "add_rmsnorm: out too small")
        if delta is not None:
            _need(out.dtype == delta.dtype, "add_rmsnorm: delta and out differ in dtype")
    _check(_lib("elementwise").ab_add_rmsnorm(_p(residual), _p(delta), _p(weight), _p(out), _dt(act), _p(rows),
                                              n, E, ctypes.c_float(eps), _stream()), "add_rmsnorm")
    return out


def add_bias(y, bias):
    """y[t,j] += bias[j] in place; bias float32."""
    _cuda(y, bias)
    N = y.shape[-1]
    _need(y.is_contiguous() and bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(),
          "add_bias: y contiguous [..,N], bias float32 [N]")
    _check(_lib("elementwise").ab_add_bias(_p(y), _dt(y), _p(bias), y.numel() // N, N, _stream()), "add_bias")
    return y


def rope_append(qkv, cos, sin, tok_pos, tok_seq, block_table, k_pages, v_pages, n_tokens, H, K, D,
                n_rot, pairing, write_cache=True, max_len=None):
    """Rotates q and k of `qkv` [T,(H+2K)D] by position and appends k, v to the pages.

    cos/sin: float32 [P, n_rot/2] or None (no rotation); pairing 0 = (2i,2i+1),
    1 = (i, n_rot/2+i).  k_pages/v_pages: [n_pages, K, page, D] of qkv's dtype.
    `max_len`: the longest sequence of the step after it (tok_pos < max_len); with it the tables'
    rows and the block table's width are checked here, else the caller guarantees tok_pos < P
    and that the block table covers tok_pos.
    """
    _cuda(qkv, cos, sin, tok_pos, tok_seq, block_table, k_pages, v_pages)
    _need(qkv.is_contiguous() and qkv.shape[-1] == (H + 2 * K) * D and qkv.numel() >= n_tokens * (H + 2 * K) * D,
          "rope_append: qkv must be contiguous [T,(H+2K)*D]")
    _i32(tok_pos, n_tokens, "tok_pos")
    _i32(tok_seq, n_tokens, "tok_seq")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(),
          "block_table must be contiguous int32 [B,W]")
    if cos is not None:
        _need(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32
              and cos.is_contiguous() and sin.is_contiguous() and cos.shape == sin.shape
              and cos.shape[-1] == n_rot // 2, "rope tables must be float32 [P, n_rot/2]")
        _need(max_len is None or max_len <= cos.shape[0],
              f"rope tables hold {cos.shape[0]} positions, the step reaches position {max_len}")
    page_size = k_pages.shape[2]
    _need(max_len is None or max_len <= block_table.shape[1] * page_size,
          f"the block table covers {block_table.shape[1] * page_size} positions, the step reaches {max_len}")
    if write_cache:
        _need(k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype and k_pages.is_contiguous()
              and v_pages.is_contiguous() and tuple(k_pages.shape[1:]) == (K, page_size, D)
              and k_pages.shape == v_pages.shape, "cache pages must be contiguous [n_pages,K,page,D] of qkv's dtype")
    _check(_lib("elementwise").ab_rope_append(
        _p(qkv), _dt(qkv), _p(cos), _p(sin), _p(tok_pos), _p(tok_seq), _p(block_table), block_table.shape[1],
        _p(k_pages), _p(v_pages), n_tokens, H, K, D, n_rot, pairing, page_size, 1 if write_cache else 0,
        _stream()), "rope_append")


def swiglu(gu, out, n_rows=None):
    """out[t,j] = silu(gate)*up from the fused, 8-row interleaved product gu [T,2F]."""
    _cuda(gu, out)
    F = gu.shape[-1] // 2
    n = gu.numel() // (2 * F) if n_rows is None else n_rows
    _need(gu.is_contiguous() and out.is_contiguous() and out.dtype == gu.dtype and out.shape[-1] == F
          and out.numel() >= n * F and gu.numel() >= n * 2 * F, "swiglu: gu [T,2F], out [T,F], same dtype")
    _need(F % 8 == 0, f"swiglu: the feed-forward width {F} must be a multiple of 8")
    _check(_lib("elementwise").ab_swiglu(_p(gu), _p(out), _dt(gu), n, F, _stream()), "swiglu")
    return out


def attention_simt(qkv, out, k_pages, v_pages, block_table, tok_pos, tok_seq, n_tokens, H, K, D, scale,
                   window=0):
    """Attention of every token over its sequence's cached keys, 32-bit arithmetic.

    qkv [T,(H+2K)D] (the q part is read), out [T,H*D].
    """
    _cuda(qkv, out, k_pages, v_pages, block_table, tok_pos, tok_seq)
    _need(qkv.is_contiguous() and out.is_contiguous() and out.dtype == qkv.dtype and k_pages.dtype == qkv.dtype,
          "attention: q, out and cache must share one dtype and be contiguous")
    _need(out.numel() >= n_tokens * H * D, "attention: out too small")
    _need(0 < D <= 256, f"attention (32-bit kernel): head size {D} is outside 1..256")
    _i32(tok_pos, n_tokens, "tok_pos")
    _i32(tok_seq, n_tokens, "tok_seq")
    page_size = k_pages.shape[2]
    _need(tuple(k_pages.shape[1:]) == (K, page_size, D) and k_pages.shape == v_pages.shape
          and k_pages.is_contiguous() and v_pages.is_contiguous(), "attention: cache pages [n_pages,K,page,D]")
    _check(_lib("attention_simt").ab_attention_simt(
        _p(qkv), qkv.shape[-1], _p(out), _dt(qkv), _p(k_pages), _p(v_pages), _p(block_table),
        block_table.shape[1], _p(tok_pos), _p(tok_seq), n_tokens, H, K, D, page_size, ctypes.c_float(scale),
        int(window or 0), _stream()), "attention_simt")
    return out


def gemm_f32(a, w, out, bias=None, n_rows=None):
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias) in true float32 (CUDA-core FMA, fixed k order)."""
    _cuda(a, w, out, bias)
    _need(a.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32,
          "gemm_f32 takes float32 tensors")
    K = a.shape[-1]
    M = a.numel() // K if n_rows is None else n_rows
    N = w.shape[0]
    _need(a.is_contiguous() and w.is_contiguous() and out.is_contiguous() and w.dim() == 2 and w.shape[1] == K
          and out.shape[-1] == N and out.numel() >= M * N and a.numel() >= M * K,
          "gemm_f32: a [M,K], w [N,K], out [M,N], contiguous")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(), "gemm_f32: bias f32 [N]")
    _check(_lib("gemm_f32").ab_gemm_f32_nt(_p(a), K, _p(w), K, _p(bias), _p(out), N, M, N, K, _stream()),
           "gemm_f32")
    return out


GEMV_MAX_ROWS = 8           # up to here the skinny-matrix kernel is the fastest (measured per shape)
GEMV_NARROW_MAX_ROWS = 16   # ... and up to here for matrices of no more 16-row slabs than the GPU has SMs
DEFER_NORM = True           # steps of up to GEMV_MAX_ROWS rows: RMS norms run inside the products around them
#                             (2048x2048: 4.1 against 5.3 us for the library, 2048x8192: 12.2 against 13.2)
# 9 to 64 rows go to the library product: the tcgen05 product with the weights on the 128-row side
# (`gemm_tc(swap=True)`) was measured against it at every shape of the 1B and 8B sizes and lost (gate|up
# with the activation 15.7-20.4 against 14.2-15.5 us, the head 95-106 against 80-98 us): a tcgen05.mma
# costs the same whatever its N, so 16 to 64 columns waste it.
TC_PERSISTENT_MIN_ROWS = 1024   # from here the persistent tcgen05 product with the SwiGLU tail beats the library
#                                 product followed by the activation kernel (16384x2048: 57.9 against 57.8 us at
#                                 1,024 rows, 100 against 120 at 2,048, 190 against 235 at 4,096)
_SM_COUNT: dict = {}


def _sm_count(device) -> int:
    n = _SM_COUNT.get(device)
    if n is None:
        n = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def gemv_bf16(x, w, out, bias=None, n_rows=None, swiglu=False, slices=None, start_early=True, owed=None,
              residual=None, norm_weight=None):
    """out[:n] = x[:n] @ w^T (+ bias) for n <= 32 rows, bfloat16 x [M,K], w [N,K].

    out bfloat16 or float32 [M,N]; with `swiglu`, w is the 8-row interleaved gate|up
    matrix [2F,K] and out is bfloat16 [M,F] = silu(gate) * up.  `start_early` off: the kernel is
    launched without programmatic dependent launch, i.e. after the kernel before it has ended (for
    the product that follows the decode attention, see csrc/launch.cuh).

    The RMS norm between two products without a kernel of its own (see csrc/gemv_bf16.cu):
    `owed` = (ss float32 [M, n_part], width, eps): x's rows still owe the division by
    sqrt(sum(ss[m]) / width + eps), which is applied to the sums.  `residual` (float32 [M,N]) with
    `norm_weight` (float32 [N]): the result is added to the residual in place, out becomes
    bf16(residual * norm_weight) and the partial sums of the residual's squares are returned as
    float32 [M, ceil(N / 16)] (the `ss` of the next product's `owed`).
    """
    _cuda(x, w, out, bias, residual, norm_weight)
    n = x.shape[0] if n_rows is None else n_rows
    K = x.shape[1]
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
          and w.dim() == 2 and w.shape[1] == K and out.is_contiguous(), "gemv_bf16: x [M,K], w [N,K] bfloat16")
    if not (0 < n <= 32 and n <= x.shape[0] and n <= out.shape[0]):
        raise KernelError(f"gemv_bf16 takes 1..32 rows, got {n}")
    if K % 8:
        raise KernelError(f"gemv_bf16: the inner size {K} must be a multiple of 8")
    ss_out = None
    if swiglu:
        _need(residual is None, "gemv_bf16: the activation and the residual epilogue exclude each other")
        _need(N % 16 == 0 and out.dtype == torch.bfloat16 and out.shape[-1] == N // 2,
              "gemv_bf16 swiglu: w [2F,K] with F a multiple of 8, out bfloat16 [M,F]")
        epi = 2
    elif residual is not None:
        _need(out.shape[-1] == N and out.dtype == torch.bfloat16, "gemv_bf16 residual: out bfloat16 [M,N]")
        _need(residual.dtype == torch.float32 and residual.is_contiguous() and residual.shape[-1] == N
              and residual.numel() >= n * N, "gemv_bf16 residual: float32 [M,N]")
        _need(norm_weight is not None and norm_weight.dtype == torch.float32 and norm_weight.numel() == N
              and norm_weight.is_contiguous(), "gemv_bf16 residual: norm weight float32 [N]")
        ss_out = torch.empty((out.shape[0], -(-N // 16)), dtype=torch.float32, device=x.device)
        epi = 3
    else:
        _need(out.shape[-1] == N and out.dtype in (torch.bfloat16, torch.float32), "gemv_bf16: out [M,N]")
        epi = 1 if out.dtype == torch.float32 else 0
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(), "gemv_bf16: bias f32 [N]")
    ss_in, n_part, inv_width, eps = None, 0, 0.0, 0.0
    if owed is not None:
        ss_in, width, eps = owed
        _cuda(ss_in)
        _need(ss_in.dtype == torch.float32 and ss_in.dim() == 2 and ss_in.is_contiguous() and ss_in.shape[0] >= n
              and width > 0, "gemv_bf16: owed sums of squares float32 [M, n_part]")
        n_part, inv_width = ss_in.shape[1], 1.0 / width
    lib = _lib("gemv_bf16")
    if slices is None:
        slices = lib.ab_gemv_bf16_slices(N, K, _sm_count(x.device))
    partials = arrivals = None
    if slices > 1:
        slabs = -(-N // 16)
        partials = torch.empty(slabs * slices * 128 * (1 if n <= 8 else 2 if n <= 16 else 4), dtype=torch.float32,
                               device=x.device)
        arrivals = _arrival_counters(x.device, slabs)
    if not start_early:
        lib.ab_pdl_hold(1)
    try:
        _check(lib.ab_gemv_bf16_norm(_p(x), _p(w), _p(bias), _p(out), _p(partials), _p(arrivals), n, N, K,
                                     out.shape[-1], epi, slices, _p(ss_in), n_part, ctypes.c_float(inv_width),
                                     ctypes.c_float(eps), _p(residual), _p(norm_weight), _p(ss_out), _stream()),
               "gemv_bf16")
    finally:
        if not start_early:
            lib.ab_pdl_hold(0)
    return out if ss_out is None else (out, ss_out)


def _prefill_tiles(ctx, G, device, rows=64):
    """Tiles of query tokens for the tensor-core prefill kernels: (sequence, first packed token),
    longest key ranges first; a tile has `rows` query rows = rows // G tokens.  Planned once per
    step, group size and tile height."""
    key = ("attention_tiles", G, rows)
    plan = ctx.extras.get(key)
    if plan is None:
        tpt = max(1, rows // G)
        tiles, start = [], 0
        for b, (q, kv) in enumerate(zip(ctx.host_q_lens, ctx.host_kv_lens)):
            for q0 in range(0, q, tpt):
                tiles.append((kv - q + min(q0 + tpt, q), b, start + q0))
            start += q
        tiles.sort(key=lambda x: -x[0])
        t = torch.tensor([[x[1] for x in tiles], [x[2] for x in tiles]], dtype=torch.int32).to(device)
        plan = (t[0].contiguous(), t[1].contiguous(), len(tiles), tpt)
        ctx.extras[key] = plan
    return plan


_ARRIVALS: dict = {}
_OUTGROWN: list = []      # scratch that was replaced by larger scratch: kept, since graphs captured earlier use it
DECODE_MAX_CLUSTER = 8           # chunks of one (sequence, head) that the decode attention merges in a cluster
USE_TCGEN05_ATTENTION = True     # prefill steps of 128 tokens or more, head size 64: the tcgen05 kernel


def _arrival_counters(device, n: int):
    """Zeroed int32 counters for the decode kernel's last-arrival merge.  Every launch leaves them
    zero again, so one buffer per device serves all launches (which run one after another in a
    stream).  It only grows outside a graph capture."""
    buf = _ARRIVALS.get(device)
    if buf is None or buf.numel() < n:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"attention: {n} arrival counters needed during graph capture, "
                              f"{0 if buf is None else buf.numel()} allocated before it")
        if buf is not None:
            _OUTGROWN.append(buf)        # captured graphs may still point at it
        buf = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _ARRIVALS[device] = buf
    return buf


_DECODE_PLANS: dict = {}


def _decode_attention_plan(pairs: int, width: int, D: int, sms: int):
    """CTA size (`small` 0, 1, 2: the CTA halved that many times, 1, 2, 4 CTAs per SM) and the number of
    chunks per sequence for the decode attention of `pairs` (sequence, KV head, head tile) triples over
    block tables `width` pages wide: the pair with the least estimated time.  The estimate is
    waves x (launch + rounds x round) + cluster, in microseconds, with constants measured on a B200
    (batch 8 and 1 at contexts of 512 to 3,800 tokens, batch 32 to 256 at 512): a CTA's launch and merge
    1.5, a round of loads and products 2.2 / 2.2 / 2.4 for the three sizes, the cluster's launch and merge
    3.2 (a second round in the same CTA costs less than a cluster of two; rounds only run for keys
    that exist, which the estimate cannot know: ties go to fewer chunks and larger CTAs)."""
    key = (pairs, width, D, sms)
    plan = _DECODE_PLANS.get(key)
    if plan is None:
        lib = _lib("attention_mma")
        best = None
        for small in (0, 1, 2):
            cap = lib.ab_attention_decode_round_keys(D, small) / 64.0        # pages per round
            slots = sms << small
            for n in range(1, DECODE_MAX_CLUSTER + 1):
                if n > 1 and n > width:
                    break
                rounds = math.ceil(-(-width // n) / cap)
                waves = -(-pairs * n // slots)
                est = waves * (1.5 + rounds * (2.2, 2.2, 2.4)[small]) + (3.2 if n > 1 else 0.0)
                if best is None or est < best[0] - 1e-9:
                    best = (est, small, n)
        plan = _DECODE_PLANS[key] = (best[1], best[2])
    return plan


_STREAM_SCRATCH: dict = {}


def _stream_scratch(device, n_partial: int, n_counters: int):
    """Scratch of the streamed decode attention's merge through memory: partial outputs, their (maximum,
    sum) pairs and zeroed arrival counters (every launch leaves them zero).  One set per device, used by
    one launch after another in a stream; it only grows outside a graph capture."""
    have = _STREAM_SCRATCH.get(device)
    if have is None or have[0].numel() < n_partial or have[2].numel() < n_counters:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"attention: scratch for {n_partial} partial sums needed during graph capture, "
                              f"{0 if have is None else have[0].numel()} allocated before it")
        n_partial = max(n_partial, 1 << 22)
        if have is not None:
            _OUTGROWN.append(have)       # captured graphs may still point at it
        have = (torch.empty(n_partial, dtype=torch.float32, device=device),
                torch.empty(max(n_partial // 8, 1 << 16), dtype=torch.float32, device=device),
                torch.zeros(max(n_counters, 1 << 16), dtype=torch.int32, device=device))
        _STREAM_SCRATCH[device] = have
    return have


def attention_stream(qkv, out, cache, ctx, H, K, D, scale, window=0, rot=None, fuse=0, pages_per_cta=8,
                     merge="memory", ring=1):
    """Decode attention that streams the cache through a ring of pages filled by TMA
    (csrc/attention_stream.cu): head sizes 64 and 128, bfloat16.  A CTA takes `pages_per_cta` pages of
    one (sequence, KV head); the chunks of a sequence are merged in chunk order, through scratch memory
    (`merge` "memory") or inside a cluster of up to 8 ("cluster").  `ring`: 0 a short ring (four CTAs per
    processor), 1 the usual one (two), 2 a deep one (one).  `fuse` as for the other decode kernel: 1 rotates q, 2 also rotates k
    and appends k, v to the cache."""
    lib = _lib("attention_stream")
    k_pages, v_pages, table = cache.k, cache.v, cache.block_table
    _cuda(qkv, out, k_pages, v_pages, table)
    T = ctx.n_tokens
    _need(lib.ab_attention_stream_supports(H, K, D) == 1, f"attention_stream: head size {D} is not 64 or 128")
    _need(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
          and qkv.is_contiguous() and out.is_contiguous() and qkv.dim() == 2 and out.numel() >= T * H * D
          and qkv.shape[-1] >= (H + (2 * K if fuse == 2 else 0)) * D and qkv.shape[0] >= T,
          "attention_stream takes contiguous bfloat16 qkv [T,(H+2K)D], out [T,H*D]")
    _need(tuple(k_pages.shape[1:]) == (K, 64, D) and k_pages.shape == v_pages.shape and k_pages.is_contiguous()
          and v_pages.is_contiguous(), "attention_stream: cache pages [n_pages,K,64,D]")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous() and table.shape[0] >= T,
          "block_table must be contiguous int32 [B,W]")
    cos, sin, n_rot, pairing = rot if (rot is not None and fuse) else (None, None, 0, 0)
    if cos is not None:
        _cuda(cos, sin)
        _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous()
              and sin.is_contiguous() and cos.shape == sin.shape and cos.shape[-1] == n_rot // 2 and n_rot % 16 == 0
              and n_rot <= D, "rope tables must be float32 [P, n_rot/2], n_rot a multiple of 16")
    _i32(ctx.tok_seq, T, "tok_seq")
    _i32(ctx.kv_len, T, "kv_len")
    order = getattr(ctx, "row_order", None)      # a permutation of the rows, longest sequence first
    if order is not None:
        _cuda(order)
        _i32(order, T, "row_order")
    width = max(int(table.shape[1]), 1)
    ppc = max(1, min(int(pages_per_cta), width))
    n_chunks = -(-width // ppc)
    kind = 0
    part_o = part_ml = arrivals = None
    if n_chunks > 1:
        if merge == "cluster" and n_chunks <= DECODE_MAX_CLUSTER:
            kind = 1
        else:
            kind = 2
            part_o, part_ml, arrivals = _stream_scratch(qkv.device, T * H * n_chunks * D, T * K * -(-(H // K) // 8))
    _tc_unchecked["attention_stream"] = True
    _check(lib.ab_attention_stream_bf16(
        _p(qkv), qkv.shape[-1], _p(out), _p(part_o), _p(part_ml), _p(arrivals), _p(k_pages), _p(v_pages),
        k_pages.shape[0], _p(table), table.shape[1], _p(ctx.tok_seq), _p(ctx.kv_len), _p(order), T, H, K, D,
        ctypes.c_float(scale), int(window or 0), ppc, n_chunks, kind, int(ring), _p(cos), _p(sin), n_rot,
        pairing, fuse, _stream()), "attention_stream")
    return out


STREAM_DECODE = True             # decode steps may take the streamed kernel (head sizes 64, 128)
STREAM_MIN_BYTES = None          # None: where it was measured to win (`_stream_pays`); a number: from that many
                                 # bytes of cache per layer, by the block table's width (0 always, inf never)


def _stream_pays(pairs: int, width: int, D: int) -> bool:
    """Whether the streamed decode attention beats the other decode kernel for `pairs` (sequence, KV head)
    pairs over block tables `width` pages wide.  Measured on a B200, each kernel with its own plan, 1 to 32
    sequences of 500 to 16,000 tokens, 8 and 32 KV heads (microseconds per layer, streamed / other): head
    size 128: it wins everywhere (one sequence of 500 tokens 6.1 / 7.8, 8 of 1,000 11.0 / 15.6, 2 of 16,000
    27 / 70); head size 64: it wins from tables of 24 pages (8 sequences of 2,000 tokens 11.0 / 14.0, 2 of 16,000
    16.8 / 33.2; a tie to 12 % worse for one or two sequences of 2,000 to 4,000), from 16 pages for up to
    four sequences (one of 1,000 tokens 5.4 / 7.3, four 6.7 / 8.1; eight are a tie at 1,000 tokens and
    lose at 800), and loses below (8 of 500 tokens 6.6 / 4.9, one 4.9 / 4.6) unless there are hundreds of
    pairs (32 sequences of 500: 9.0 / 10.1)."""
    if STREAM_MIN_BYTES is not None:
        return pairs * width * 64 * D * 4 >= STREAM_MIN_BYTES
    return D == 128 or width >= 24 or (width >= 16 and pairs <= 32) or pairs * width * 64 * D * 4 >= 30e6


def _stream_plan(rows: int, H: int, K: int, D: int, width: int, sms: int):
    """Whether the streamed decode attention should take a step of `rows` sequences whose block table is
    `width` pages wide, and how: None, or (pages per CTA, merge, ring).  Measured on a B200 against the
    other decode kernel at its best plan (microseconds per layer): 64 sequences of 530 tokens, 8 KV heads
    of 64: 15.4 against 17.5; of 2,000 tokens: 48.4 against 55.3; 64 sequences of 128 to 2,048 tokens, 8
    KV heads of 128: 63.1 against 100.9; 8 sequences of 16 to 1,024 tokens, 32 KV heads of 128: 17.9
    against 31.6; 8 sequences of 3,800 tokens, 8 heads of 64: 15.5 against 18.4.  Where little is read it loses
    at head size 64 (8 sequences of 640 tokens: 6.9 against 5.1; one sequence: 5.4 against 4.75), hence
    `_stream_pays`.  One CTA per (sequence, KV head) is best once there are more of those than processors;
    fewer are cut into chunks that a cluster merges; many CTAs of few pages take the short ring."""
    if not STREAM_DECODE or D not in (64, 128):
        return None
    pairs = rows * K * -(-(H // K) // 8)
    if not _stream_pays(pairs, width, D):
        return None
    want = -(-3 * sms // (2 * pairs))
    if want > DECODE_MAX_CLUSTER and width >= 8 * DECODE_MAX_CLUSTER:
        # few long sequences: more chunks than a cluster holds, merged through memory by the CTA that arrives
        # last, so that there are about 7/4 CTAs per processor, none with fewer than 4 pages (one sequence
        # of 30,000 tokens, 8 KV heads of 64: 18.9 us per layer with 32 chunks against 30.7 with a cluster's 8)
        chunks = max(1, min(-(-7 * sms // (4 * pairs)), width // 4, 64))
        return -(-width // chunks), "memory", 1
    chunks = max(1, min(DECODE_MAX_CLUSTER, want, width))
    ppc = -(-width // chunks)
    ring = 0 if (pairs * chunks > 2 * sms and ppc <= 16) else 1
    return ppc, "cluster", ring


def _attention_decode(qkv, out, cache, ctx, H, K, D, scale, window, rot=None, fuse=0):
    """Decode attention of one token per row of the batch: the kernel that fits the step's size."""
    plan = _stream_plan(ctx.n_tokens, H, K, D, max(int(cache.block_table.shape[1]), 1), _sm_count(qkv.device))
    if plan is not None:
        return attention_stream(qkv, out, cache, ctx, H, K, D, scale, window, rot, fuse, pages_per_cta=plan[0],
                                merge=plan[1], ring=plan[2])
    return _attention_decode_mma(qkv, out, cache, ctx, H, K, D, scale, window, rot, fuse)


def _attention_decode_mma(qkv, out, cache, ctx, H, K, D, scale, window, rot=None, fuse=0):
    """Decode attention: a CTA per (sequence, KV head, chunk of pages).  With few (sequence, head)
    pairs a CTA is large and a long table is cut into 2 to 8 chunks that are merged inside a
    thread-block cluster; with more pairs than processors the CTAs are smaller (several per
    processor) and each walks its whole table in rounds.
    `fuse` 1: the kernel also rotates q; 2: it rotates q and k and appends k, v to the cache."""
    lib = _lib("attention_mma")
    k_pages, v_pages, table = cache.k, cache.v, cache.block_table
    T = ctx.n_tokens
    cos, sin, n_rot, pairing = rot if (rot is not None and fuse) else (None, None, 0, 0)
    if cos is not None:
        _cuda(cos, sin)
        _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous()
              and sin.is_contiguous() and cos.shape == sin.shape and cos.shape[-1] == n_rot // 2 and n_rot % 16 == 0
              and n_rot <= D, "rope tables must be float32 [P, n_rot/2], n_rot a multiple of 16")
    width = max(int(table.shape[1]), 1)
    small, n_chunks = _decode_attention_plan(T * K * -(-(H // K) // 8), width, D, _sm_count(qkv.device))
    pages_per_cta = -(-width // n_chunks)
    _i32(ctx.tok_seq, T, "tok_seq")
    _i32(ctx.kv_len, ctx.n_seqs, "kv_len")
    _check(lib.ab_attention_decode_rope_bf16(
        _p(qkv), qkv.shape[-1], _p(out), None, None, None, _p(k_pages), _p(v_pages), _p(table), table.shape[1],
        _p(ctx.tok_seq), _p(ctx.kv_len), T, H, K, D, ctypes.c_float(scale), int(window or 0), pages_per_cta,
        n_chunks, small, _p(cos), _p(sin), n_rot, pairing, fuse, _stream()), "attention_decode")
    return out


def attention_mma(qkv, out, cache, ctx, H, K, D, scale, window=0):
    """Tensor-core attention (bfloat16) over the paged cache; prefill or decode by the step's kind."""
    k_pages, v_pages, table = cache.k, cache.v, cache.block_table
    _cuda(qkv, out, k_pages, v_pages, table)
    T = ctx.n_tokens
    _need(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
          and qkv.is_contiguous() and out.is_contiguous(), "attention_mma takes contiguous bfloat16 tensors")
    _need(D % 16 == 0 and 0 < D <= 256 and H % K == 0 and H // K <= 64,
          f"attention_mma: head size {D} (multiples of 16 up to 256) or group size {H // K} (up to 64) not supported")
    _need(qkv.shape[-1] == (H + 2 * K) * D and out.numel() >= T * H * D, "attention_mma: qkv [T,(H+2K)D], out [T,H*D]")
    page = k_pages.shape[2]
    _need(page == 64 and tuple(k_pages.shape[1:]) == (K, 64, D) and k_pages.shape == v_pages.shape
          and k_pages.is_contiguous() and v_pages.is_contiguous(), "attention_mma: cache pages [n_pages,K,64,D]")
    lib = _lib("attention_mma")
    if ctx.is_decode:
        _i32(ctx.tok_seq, T, "tok_seq")
        return _attention_decode(qkv, out, cache, ctx, H, K, D, scale, window)
    _i32(ctx.tok_pos, T, "tok_pos")
    _i32(ctx.cu_q, ctx.n_seqs + 1, "cu_q")
    if USE_TCGEN05_ATTENTION and T >= 128 and qkv.shape[0] >= T:
        tc = _lib("attention_tc")
        if tc.ab_attention_prefill_tc_supports(H, K, D):
            _tc_unchecked["attention_tc"] = True
            tile_seq, tile_q0, n_tiles, _ = _prefill_tiles(ctx, H // K, qkv.device, rows=128)
            _check(tc.ab_attention_prefill_tc(
                _p(qkv), T, _p(out), _p(k_pages), _p(v_pages), k_pages.shape[0], _p(table), table.shape[1],
                _p(ctx.tok_pos), _p(ctx.cu_q), _p(tile_seq), _p(tile_q0), n_tiles, H, K, D, ctypes.c_float(scale),
                int(window or 0), _stream()), "attention_prefill_tc")
            return out
    tile_seq, tile_q0, n_tiles, tpt = _prefill_tiles(ctx, H // K, qkv.device)
    _check(lib.ab_attention_prefill_bf16(
        _p(qkv), qkv.shape[-1], _p(out), _p(k_pages), _p(v_pages), _p(table), table.shape[1], _p(ctx.tok_pos),
        _p(ctx.cu_q), _p(tile_seq), _p(tile_q0), n_tiles, tpt, H, K, D, ctypes.c_float(scale), int(window or 0),
        _stream()), "attention_prefill")
    return out


def attention(qkv, out, cache, ctx, H, K, D, scale, window=0):
    """Attention of the step's tokens over the paged cache (`cache`: a KVLayerView).

    bfloat16 with a head size in steps of 16 up to 256: the tensor-core kernels; everything
    else (the 32-bit path, other head sizes up to 256): the 32-bit kernel."""
    if qkv.dtype == torch.bfloat16 and D % 16 == 0 and D <= 256 and H // K <= 64:
        return attention_mma(qkv, out, cache, ctx, H, K, D, scale, window)
    return attention_simt(qkv, out, cache.k, cache.v, cache.block_table, ctx.tok_pos, ctx.tok_seq,
                          ctx.n_tokens, H, K, D, scale, window)


FUSE_ROPE_DECODE = True          # decode steps: rotation and append inside the attention kernel


def rope_attention(qkv, out, cache, ctx, H, K, D, scale, window=0, rot=None, write_cache=True):
    """Position rotation of q and k (`rot` = (cos, sin, n_rot, pairing) or None), append of k and v to
    the cache (unless `write_cache` is off: a layer that reads another layer's cache), then attention
    of the step's tokens over the cache.  Decode steps in bfloat16 do all of it in one kernel; everything else runs the rotation kernel and then `attention`."""
    cos, sin, n_rot, pairing = rot if rot is not None else (None, None, 0, 0)
    T = ctx.n_tokens
    max_len = getattr(ctx, "max_kv_len", None)
    if cos is not None and max_len is not None:
        _need(max_len <= cos.shape[0], f"rope tables hold {cos.shape[0]} positions, the step reaches position {max_len}")
    if (FUSE_ROPE_DECODE and ctx.is_decode and qkv.dtype == torch.bfloat16 and D % 16 == 0 and D <= 256
            and H // K <= 64 and n_rot % 16 == 0):
        _cuda(qkv, out, cache.k, cache.v, cache.block_table)
        _need(out.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16 and qkv.is_contiguous()
              and out.is_contiguous() and qkv.shape[-1] == (H + 2 * K) * D and out.numel() >= T * H * D
              and H % K == 0, "rope_attention takes contiguous bfloat16 qkv [T,(H+2K)D], out [T,H*D]")
        _need(tuple(cache.k.shape[1:]) == (K, 64, D) and cache.k.shape == cache.v.shape and cache.k.is_contiguous()
              and cache.v.is_contiguous(), "rope_attention: cache pages [n_pages,K,64,D]")
        return _attention_decode(qkv, out, cache, ctx, H, K, D, scale, window, rot, 2 if write_cache else 1)
    rope_append(qkv, cos, sin, ctx.tok_pos, ctx.tok_seq, cache.block_table, cache.k, cache.v, T, H, K, D, n_rot,
                pairing, write_cache=write_cache, max_len=max_len)
    return attention(qkv, out, cache, ctx, H, K, D, scale, window)


def defers_norm(n_rows: int, width: int) -> bool:
    """Whether the product before a norm of a `width`-wide stream can leave `n_rows` rows prepared for
    the product after it (both must be the skinny product, see `gemv_bf16`)."""
    return DEFER_NORM and 0 < n_rows <= GEMV_MAX_ROWS and width % 8 == 0


def owed_norm_pays(n_rows: int, out_features: int, in_features: int, device) -> bool:
    """Whether the product [out_features, in_features] after a norm should finish the norm itself in a
    step of `n_rows` rows: only where its 16-row slabs are all resident at once (two CTAs per
    processor).  A grid of several waves loses more by the added tail of every CTA than the norm's
    kernel costs (measured, see csrc/gemv_bf16.cu)."""
    return (defers_norm(n_rows, in_features) and -(-out_features // 16) <= 2 * _sm_count(device))


def linear_bf16(x, w, out, n_rows=None, bias=None, start_early=True, owed=None):
    """out[:n] = x[:n] @ w^T (+ bias) for bfloat16 x [M,K], w [N,K]; out bfloat16 or float32 [M,N].

    Up to GEMV_MAX_ROWS rows (decode steps; GEMV_NARROW_MAX_ROWS for narrow matrices): the
    skinny-matrix kernel, which reads the weights once.  More rows: the library matrix product (as
    the reference uses BLAS)."""
    _cuda(x, w, out)
    n = x.shape[0] if n_rows is None else n_rows
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear_bf16 takes bfloat16 inputs")
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and out.shape[-1] == w.shape[0],
          "linear_bf16: x [M,K], w [N,K], out [M,N]")
    if x.shape[1] % 8 == 0 and (n <= GEMV_MAX_ROWS or (n <= GEMV_NARROW_MAX_ROWS
                                                       and -(-w.shape[0] // 16) <= _sm_count(x.device))):
        return gemv_bf16(x, w, out, bias=bias, n_rows=n, start_early=start_early, owed=owed)
    _need(owed is None, "linear_bf16: only the skinny product finishes a norm that its input owes")
    xs, ys = (x, out) if n == x.shape[0] == out.shape[0] else (x[:n], out[:n])
    if out.dtype == torch.float32:
        torch.mm(xs, w.t(), out_dtype=torch.float32, out=ys)
    else:
        torch.mm(xs, w.t(), out=ys)
    _mark("library product")
    if bias is not None:
        add_bias(ys, bias)
    return out


def repeat_penalty(logits, recent, penalty):
    """In place: for each distinct token of a row's window (int32 [B,R], -1 = unused),
    l > 0 -> l / penalty, else l * penalty."""
    _cuda(logits, recent)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(),
          "repeat_penalty: logits float32 [B,V]")
    _need(recent.dtype == torch.int32 and recent.dim() == 2 and recent.is_contiguous()
          and recent.shape[0] == logits.shape[0], "repeat_penalty: recent int32 [B,R]")
    _check(_lib("sampling").ab_repeat_penalty(_p(logits), _p(recent), logits.shape[0], recent.shape[1],
                                              logits.shape[1], ctypes.c_float(penalty), _stream()),
           "repeat_penalty")
    return logits


def sample(logits, out, temperature, top_k, top_p, seed, streams, steps, seed_dev=None):
    """One token per row of float32 logits [B,V] into out int32 [B].

    temperature <= 0: first index of the maximum.  Else top_k (<= 0: all), top_p
    (>= 1: all), and a draw with Philox(seed; stream, step) per row.  `seed_dev` (int32 [2]: low
    and high word, on the device) replaces `seed` when given.
    """
    _cuda(logits, out, streams, steps)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(),
          "sample: logits float32 [B,V]")
    B, V = logits.shape
    _i32(out, B, "out")
    _i32(streams, B, "streams")
    _i32(steps, B, "steps")
    if seed_dev is not None:
        _cuda(seed_dev)
        _i32(seed_dev, 2, "seed_dev")
    _check(_lib("sampling").ab_sample(_p(logits), B, V, _p(out), ctypes.c_float(temperature), int(top_k),
                                      ctypes.c_float(top_p), ctypes.c_uint64(int(seed) & (2**64 - 1)),
                                      _p(seed_dev), _p(streams), _p(steps), _stream()), "sample")
    return out


def decode_advance(tokens, tok_pos, kv_len, rng_step, tok_seq, sampled, recent, recent_pos, window,
                   history, counter, n_rows, host_ring=None):
    """Feeds the sampled tokens back as the next step's inputs (all int32, on the device); see the kernel.
    `host_ring`: pinned host memory int32 [R, rows]; the step's tokens are also written to its row
    counter % R, by the kernel itself."""
    _cuda(tokens, tok_pos, kv_len, rng_step, tok_seq, sampled, recent, recent_pos, history, counter)
    for t, name in ((tokens, "tokens"), (tok_pos, "tok_pos"), (kv_len, "kv_len"), (rng_step, "rng_step"),
                    (tok_seq, "tok_seq"), (sampled, "sampled")):
        _i32(t, n_rows, name)
    hist_len = 0
    if history is not None:
        _need(history.dtype == torch.int32 and history.is_contiguous() and history.shape[1] == n_rows
              and counter is not None and counter.dtype == torch.int32, "decode_advance: history int32 [L, rows]")
        hist_len = history.shape[0]
    if recent is not None:
        _need(recent.dtype == torch.int32 and recent.is_contiguous() and recent.numel() >= n_rows * window
              and recent_pos is not None, "decode_advance: recent int32 [rows, window]")
        _i32(recent_pos, n_rows, "recent_pos")
    ring_len = 0
    if host_ring is not None:
        _need(host_ring.device.type == "cpu" and host_ring.is_pinned() and host_ring.dtype == torch.int32
              and host_ring.is_contiguous() and host_ring.dim() == 2 and host_ring.shape[1] == n_rows
              and counter is not None, "decode_advance: host_ring pinned int32 [R, rows], with a counter")
        ring_len = host_ring.shape[0]
    _check(_lib("elementwise").ab_decode_advance(
        _p(tokens), _p(tok_pos), _p(kv_len), _p(rng_step), _p(tok_seq), _p(sampled), _p(recent), _p(recent_pos),
        int(window), _p(history), _p(counter), hist_len, _p(host_ring), ring_len, n_rows, _stream()),
        "decode_advance")


def gemm_tc(x, w, out, bias=None, n_rows=None, swiglu=False, swap=None, bn=None, slices=None, persistent=True,
            pair=None):
    """out[:n] = x[:n] @ w^T (+ bias) on the tcgen05 tensor cores (TMA-fed, TMEM accumulators).

    x [M,K], w [N,K] bfloat16; out bfloat16 or float32 [M,N]; with `swiglu`, w is the 8-row
    interleaved gate|up matrix and out is bfloat16 [M, N/2].  `swap` puts the weights on the
    128-row side of the MMA (the batch, up to 256 rows, becomes the columns): the shape for decode
    steps.  `bn` is the MMA's column count per tile, `slices` the number of K slices.  Without `swap`,
    256-wide tiles and one slice run as the persistent kernel (one CTA per SM walks the tiles) unless
    `persistent` is off; `pair` chooses its form on pairs of processors (tiles of 256 x 256,
    `tcgen05.mma.cta_group::2`; default: `TC_PAIR`).
    """
    _cuda(x, w, out, bias)
    n = x.shape[0] if n_rows is None else n_rows
    K, N = x.shape[1], w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
          and w.dim() == 2 and w.shape[1] == K and out.is_contiguous(), "gemm_tc: x [M,K], w [N,K] bfloat16")
    _need(K % 8 == 0, f"gemm_tc: the inner size {K} must be a multiple of 8")
    _need(x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0, "gemm_tc: operands must be 16-byte aligned")
    _need(0 < n <= x.shape[0] and n <= out.shape[0], "gemm_tc: row count")
    if swap is None:
        swap = n <= 64
    if bn is None:
        bn = (16 if n <= 16 else 32 if n <= 32 else 64 if n <= 64 else 128 if n <= 128 else 256) if swap else 256
    _need(bn in (16, 32, 64, 128, 256), "gemm_tc: bn must be 16, 32, 64, 128 or 256")
    if swiglu:
        _need(N % 16 == 0 and out.dtype == torch.bfloat16 and out.shape[-1] == N // 2,
              "gemm_tc swiglu: w [2F,K] with F a multiple of 8, out bfloat16 [M,F]")
        epi = 2
    else:
        _need(out.shape[-1] == N and out.dtype in (torch.bfloat16, torch.float32), "gemm_tc: out [M,N]")
        epi = 1 if out.dtype == torch.float32 else 0
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(), "gemm_tc: bias f32 [N]")
    _tc_unchecked["gemm_tc"] = True
    if not swap and bn == 256 and slices in (None, 1) and persistent:
        # many rows: the persistent form (tails under the next tile's main loop)
        lib = _lib("gemm_tc")
        run = lib.ab_gemm_tc_pair if (TC_PAIR if pair is None else pair) else lib.ab_gemm_tc_persistent
        _check(run(_p(x), _p(w), _p(bias), _p(out), n, N, K, out.shape[-1], epi, _stream()), "gemm_tc")
        return out
    rows_a, rows_b = (N, n) if swap else (n, N)
    tiles = -(-rows_a // 128) * -(-rows_b // bn)
    if slices is None:
        slices = max(1, min(-(-2 * _sm_count(x.device) // tiles), K // 1024)) if swap else 1
    partials = arrivals = None
    if slices > 1:
        partials = torch.empty(tiles * slices * 128 * bn, dtype=torch.float32, device=x.device)
        arrivals = _arrival_counters(x.device, tiles)
    _check(_lib("gemm_tc").ab_gemm_tc(_p(x), _p(w), _p(bias), _p(out), _p(partials), _p(arrivals), n, N, K,
                                      out.shape[-1], epi, 1 if swap else 0, bn, slices, _stream()), "gemm_tc")
    return out


# The persistent product on pairs of processors (`tcgen05.mma.cta_group::2`, see `gemm_tc`).  Measured on a
# B200 against the form with one processor per tile: gate|up with the activation 2048 x 16384 x 2048 101.6
# against 100.9 us, 4797 x 22016 x 4096 587 against 602, plain 16384 x 4096 x 14336 1,307 against 1,412 us
# (library 1,258); whole prompt steps: 1B shape 2,048 tokens 4.35 ms either way, the 7B workload's 4,797 tokens
# 55.0 against 56.2 ms, the 8B workload's 76,771 tokens 1.00 against 1.07 s (it moves a third less through the
# shared memory, which under the power cap is worth more than the kernel alone shows).
TC_PAIR = True

# kernels that wait on barriers with a limit, launched since the last check
_tc_unchecked = {"gemm_tc": False, "attention_tc": False, "attention_stream": False}


def check_tc_status() -> None:
    """Raises `KernelError` if a kernel that waits on barriers with a limit (the tcgen05 kernels, the
    streamed decode attention), launched since the last call, gave up a wait (its output is then
    unfinished).  Call it where the stream has just been synchronised: it reads one word per library
    from the device, and nothing when no such kernel ran."""
    for name, read in (("gemm_tc", gemm_tc_status), ("attention_tc", attention_tc_status),
                       ("attention_stream", attention_stream_status)):
        if _tc_unchecked[name]:
            _tc_unchecked[name] = False
            code = read()
            if code:
                raise KernelError(f"a kernel of {name} gave up waiting on a barrier (code {code}); "
                                  "the results of the steps since the last check are not valid")


def gemm_tc_status() -> int:
    """0, or the code left by a tcgen05 kernel that gave up waiting on a barrier (synchronises)."""
    return _lib("gemm_tc").ab_gemm_tc_status()


def attention_tc_status() -> int:
    """0, or the code left by a tcgen05 attention kernel that gave up waiting on a barrier (synchronises)."""
    return _lib("attention_tc").ab_attention_tc_status()


def attention_stream_status() -> int:
    """0, or the code left by a streamed decode attention kernel that gave up waiting on a barrier (synchronises)."""
    return _lib("attention_stream").ab_attention_stream_status()
