#!/usr/bin/env python3
"""Outputs of jtiro232/Alpacca's own model code on tiny random models (CPU).

usage: python tests/golden/make_golden.py /path/to/Alpacca

Builds `alpacca.model.Model` in memory (no GGUF file, no tokenizer) with the
weights of `tests/tiny.py`, feeds one prompt token by token through its
`forward()` (alpacca/model.py:439-445) and keeps the logits of every position,
and once more as one batch through `forward_batch()` (:469-518) for the last
position.  The arrays go to `tests/golden/<name>.npz`; the test
`tests/test_plain_vs_golden.py` compares `tests/plain_llama.py` with them.

The reference has no frequency scaling: the scaled frequencies (computed here
with the same published formula as the plain implementation) are written over
its `_rope_inv_freq` before its tables are built (alpacca/model.py:352-356),
so everything after the table of frequencies is the reference's own
arithmetic.  It has no bias on the output projection or in the feed-forward
either; configuration C is run with those biases zero.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import plain_llama as plain  # noqa: E402
import tiny  # noqa: E402

CASES = {"tiny_a": (tiny.TINY_A, 0, 17), "tiny_b": (tiny.TINY_B, 1, 70), "tiny_c": (tiny.TINY_C, 2, 40)}


def golden_weights(cfg, seed):
    w = tiny.make_weights(cfg, seed)
    for name in w:
        if name.endswith("o_proj.bias") or ("mlp." in name and name.endswith(".bias")):
            w[name][...] = 0.0
    return w


def build_reference(cfg, w, ref_root):
    sys.path.insert(0, str(ref_root))
    from alpacca.model import Hyperparams, Layer, Model

    E, H = cfg["hidden_size"], cfg["num_attention_heads"]
    D = cfg.get("head_dim") or E // H
    hp = Hyperparams(
        arch="llama", n_layer=cfg["num_hidden_layers"], n_embd=E, n_head=H,
        n_kv=cfg.get("num_key_value_heads") or H, n_ff=cfg["intermediate_size"],
        n_vocab=cfg["vocab_size"], n_ctx_train=cfg["max_position_embeddings"], head_dim=D,
        n_rot=cfg.get("rotary_dim") or D, rms_eps=cfg["rms_norm_eps"], rope_base=cfg["rope_theta"],
        rope_style={"llama": "norm", "neox": "neox"}[cfg["rope_pairing"]])
    m = Model(hp, None)
    m.tok_embd = w["model.embed_tokens.weight"]
    for i in range(hp.n_layer):
        p = f"model.layers.{i}."
        ly = Layer()
        ly.attn_norm = w[p + "input_layernorm.weight"]
        ly.wq, ly.wk, ly.wv, ly.wo = (w[p + f"self_attn.{n}_proj.weight"] for n in "qkvo")
        ly.bq, ly.bk, ly.bv = (w.get(p + f"self_attn.{n}_proj.bias") for n in "qkv")
        ly.ffn_norm = w[p + "post_attention_layernorm.weight"]
        ly.w_gate, ly.w_up, ly.w_down = (w[p + f"mlp.{n}_proj.weight"] for n in ("gate", "up", "down"))
        m.layers.append(ly)
    m.out_norm = w["model.norm.weight"]
    m.output = m.tok_embd if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    m.n_ctx = cfg["max_position_embeddings"]
    scaled = plain.scale_inv_freq(plain.rope_inv_freq(hp.n_rot, hp.rope_base), cfg.get("rope_scaling"))
    m._rope_inv_freq = scaled.astype(np.float32)
    m._rope_cos = None
    m._init_cache()
    return m


def main():
    ref_root = Path(sys.argv[1])
    for name, (cfg, seed, n_tok) in CASES.items():
        w = golden_weights(cfg, seed)
        ids = tiny.prompt_tokens(cfg, n_tok, seed)
        m = build_reference(cfg, w, ref_root)
        rows = np.stack([np.asarray(m.forward(t), np.float32) for t in ids])
        m.reset()
        last = np.asarray(m.forward_batch(ids), np.float32)
        np.savez_compressed(HERE / f"{name}.npz", tokens=np.asarray(ids, np.int32),
                            logits_token_by_token=rows, logits_batch_last=last)
        print(name, rows.shape, float(np.abs(rows[-1] - last).max()))


if __name__ == "__main__":
    main()
