"""Configurations drawn at random (from a fixed seed each) through the engine against the plain
implementation, in 32-bit and in bfloat16: head sizes in steps of 16 up to 256, one to eighty heads in
groups of 1 to 16, widths and vocabularies that are odd, even or multiples of 8, biases, tied heads, both
pairings, rotation of a part of the head, every kind of frequency scaling.  Each is stepped whole, as a
batch of unequal prompts that are then fed on one token at a time (one sequence ends early), and as a
prompt in two chunks whose second lands on a cache that holds the first."""
import random

import pytest
import torch

import plain_llama as plain
import tiny
from helpers import check_logits

pytestmark = pytest.mark.gpu


def draw(i: int):
    rng = random.Random(7000 + i)
    D = rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 160, 192, 256])
    K = rng.choice([1, 1, 2, 3, 5])
    G = rng.choice([1, 2, 3, 4, 4, 7, 8, 12, 16])
    while K * G * D > 3072:
        G = max(1, G // 2)
    cfg = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": rng.choice([1, 2, 3]),
           "hidden_size": rng.choice([24, 40, 56, 72, 100, 136, 200, 264, 36, 50, 37]),
           "num_attention_heads": K * G, "num_key_value_heads": K, "head_dim": D,
           "intermediate_size": rng.choice([24, 40, 104, 264, 520, 1000]),
           "vocab_size": rng.choice([97, 300, 1003, 2049, 4099]), "max_position_embeddings": 512,
           "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-4]), "rope_theta": rng.choice([10000.0, 500000.0, 777.0]),
           "rope_pairing": rng.choice(["llama", "neox"]),
           "rope_scaling": rng.choice([None, {"rope_type": "linear", "factor": 2.0},
                                       {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                        "high_freq_factor": 4.0, "original_max_position_embeddings": 64}]),
           "tie_word_embeddings": rng.random() < 0.5, "attention_bias": rng.random() < 0.3,
           "mlp_bias": rng.random() < 0.3, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2}
    if rng.random() < 0.3:
        cfg["rotary_dim"] = rng.choice([d for d in (8, 16, 32, 64) if d <= D])
    return cfg, rng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("i", range(16))
def test_a_configuration_drawn_at_random(tmp_path, i, dtype):
    from alpacca_b200.engine import Engine, StepEntry
    from alpacca_b200.engine.loading import load_model_dir, write_random_model_dir
    cfg, rng = draw(i)
    what = (f"{cfg['num_attention_heads']}/{cfg['num_key_value_heads']} heads of {cfg['head_dim']}, width "
            f"{cfg['hidden_size']}, inner {cfg['intermediate_size']}, vocabulary {cfg['vocab_size']}")
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    d = write_random_model_dir(tmp_path / "m", cfg, 50 + i, dtype=dt, std=0.1)     # sharp attention
    pm = plain.PlainLlama.from_dir(str(d))
    eng = Engine(load_model_dir(d, dtype=dtype, device="cuda"), max_tokens=64 * 24, max_slots=6)
    lens = [rng.choice([1, 5, 33, 64, 65, 127, 129, 200, 300]) for _ in range(3)]
    toks = [tiny.prompt_tokens(cfg, n + 8, 7 * i + j) for j, n in enumerate(lens)]
    want = [pm.logits(t) for t in toks]

    s = eng.alloc_slot()
    got = eng.step([StepEntry(s, toks[0], list(range(len(toks[0]))))]).cpu().numpy()
    check_logits(got, want[0], dtype, f"{what}: whole")
    eng.free_slot(s)

    slots = [eng.alloc_slot() for _ in toks]
    got = eng.step([StepEntry(s, t[:n], [n - 1]) for s, t, n in zip(slots, toks, lens)]).cpu().numpy()
    for j in range(3):
        check_logits(got[j], want[j][lens[j] - 1], dtype, f"{what}: prompt {j} of the batch")
    live = [0, 1, 2]
    for p in range(8):
        if p == 3:
            live.remove(1)
            eng.free_slot(slots[1])
        got = eng.step([StepEntry(slots[j], [toks[j][lens[j] + p]], [0]) for j in live]).cpu().numpy()
        for r, j in enumerate(live):
            check_logits(got[r], want[j][lens[j] + p], dtype, f"{what}: token {p} of sequence {j} fed alone")
    for j in live:
        eng.free_slot(slots[j])

    n = len(toks[2])
    a = rng.randrange(1, n - 1)
    s = eng.alloc_slot()
    eng.step([StepEntry(s, toks[2][:a], [])])
    got = eng.step([StepEntry(s, toks[2][a:], list(range(n - a)))]).cpu().numpy()
    check_logits(got, want[2][a:], dtype, f"{what}: second chunk from {a} of {n}")
    eng.free_slot(s)
    eng.cache.check()
    eng.wait()
