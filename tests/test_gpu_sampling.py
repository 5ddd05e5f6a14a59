"""The sampling kernels against the plain sampler."""
import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu


def gpu_sample(logits, temperature, top_k, top_p, seed, streams, steps):
    from alpacca_b200 import ops
    l = torch.tensor(np.asarray(logits, np.float32)).cuda()
    out = torch.empty(l.shape[0], dtype=torch.int32, device="cuda")
    ops.sample(l, out, temperature, top_k, top_p, seed,
               torch.tensor(streams, dtype=torch.int32).cuda(), torch.tensor(steps, dtype=torch.int32).cuda())
    return out.tolist()


def agrees(row, tok, temperature, top_k, top_p, u):
    """The plain sampler's token for u, allowing for rounding of the running sums at a boundary."""
    return tok in {plain.sample(row, temperature, top_k, top_p, min(max(u + d, 0.0), 1 - 1e-9))
                   for d in (0.0, -2e-6, 2e-6)}


@pytest.mark.parametrize("V", [50, 1003, 128256])
def test_greedy_first_index_of_the_maximum(V):
    rng = np.random.default_rng(V)
    l = rng.standard_normal((5, V)).astype(np.float32)
    l[1, [7, V - 1]] = 9.0         # a tie: the lower index wins
    l[2, V - 1] = 9.0              # the very last entry
    l[3, :] = -3.0                 # all equal
    got = gpu_sample(l, 0.0, 40, 0.9, 1, [0] * 5, [0] * 5)
    assert got == [int(np.argmax(r)) for r in l] and got[1] == 7 and got[2] == V - 1 and got[3] == 0


@pytest.mark.parametrize("V", [50, 1003, 128256])
@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 0, 1.0), (1.0, 40, 1.0), (0.7, 0, 0.9), (0.8, 40, 0.95),
                                                     (1.5, 5, 0.5), (0.3, 1, 1.0), (2.0, 1000, 0.99)])
def test_draws_agree_with_the_plain_sampler(V, temperature, top_k, top_p):
    rng = np.random.default_rng(V + top_k)
    B = 16
    l = (rng.standard_normal((B, V)) * 2.5).astype(np.float32)
    l[3, rng.integers(0, V, 12)] = l[3].max()            # ties at the top
    l[4] = np.round(l[4])                                # many ties everywhere
    seed, streams, steps = 1234567890123, list(range(B)), [3 * b for b in range(B)]
    got = gpu_sample(l, temperature, top_k, top_p, seed, streams, steps)
    for b in range(B):
        u = plain.uniform(seed, streams[b], steps[b])
        assert agrees(l[b], got[b], temperature, top_k, top_p, u), \
            f"row {b}: kernel {got[b]}, plain {plain.sample(l[b], temperature, top_k, top_p, u)} (u={u})"


def test_a_row_does_not_depend_on_the_batch():
    rng = np.random.default_rng(0)
    l = (rng.standard_normal((8, 1003)) * 2).astype(np.float32)
    whole = gpu_sample(l, 0.9, 50, 0.9, 42, list(range(8)), [5] * 8)
    for b in (0, 3, 7):
        assert gpu_sample(l[b:b + 1], 0.9, 50, 0.9, 42, [b], [5]) == [whole[b]]


def test_frequencies_follow_the_distribution():
    l = np.array([[2.0, 1.0, 0.0, -1.0, 1.0, -30.0]], np.float32)
    n = 4000
    rows = np.repeat(l, n, axis=0)
    got = np.array(gpu_sample(rows, 1.0, 0, 1.0, 7, [0] * n, list(range(n))))
    p = np.exp(l[0] - l[0].max())
    p /= p.sum()
    freq = np.bincount(got, minlength=6) / n
    assert np.abs(freq - p).max() < 0.03 and freq[5] == 0


def test_repeat_penalty():
    from alpacca_b200 import ops
    l = torch.tensor([[2.0, -2.0, 1.0, 4.0], [1.0, 1.0, 1.0, 1.0]]).cuda()
    recent = torch.tensor([[0, 1, 0, -1], [3, -1, -1, -1]], dtype=torch.int32).cuda()
    ops.repeat_penalty(l, recent, 2.0)
    assert l.tolist() == [[1.0, -4.0, 1.0, 4.0], [1.0, 1.0, 1.0, 0.5]]


def test_device_sampler_keeps_state():
    from alpacca_b200.sampling import DeviceSampler, SamplerParams
    s = DeviceSampler(SamplerParams(temperature=0.0, repeat_penalty=10.0, repeat_last_n=2, seed=1), "cuda")
    st = s.new_state(0, [1, 2, 3])
    assert st.recent == [2, 3]
    l = torch.tensor([[0.1, 0.2, 5.0, 6.0, 0.7]]).cuda()
    assert s.sample(l.clone(), [st]) == [4]          # 2 and 3 are penalised to .5 and .6
    assert st.recent == [3, 4] and st.step == 1
    assert s.sample(l.clone(), [st]) == [2]          # now 3 and 4 are
