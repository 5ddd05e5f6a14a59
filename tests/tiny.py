"""Tiny configurations and deterministic weights for the tests.

The two configurations differ in every size and option: layers, width, heads,
KV heads (MHA against groups of 3), head size, feed-forward width, vocabulary,
rope base, pairing, frequency scaling, eps, tied or untied head, biases,
maximum position.  `make_weights` depends on nothing but integer arithmetic
(splitmix64 and Box-Muller), so the golden outputs stay reproducible whatever
NumPy's own generators do in later versions.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 4,
    "head_dim": 16,
    "intermediate_size": 160,
    "vocab_size": 256,
    "max_position_embeddings": 128,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "rope_pairing": "llama",
    "rope_scaling": None,
    "tie_word_embeddings": False,
    "attention_bias": False,
    "mlp_bias": False,
    "hidden_act": "silu",
    "bos_token_id": 1,
    "eos_token_id": 2,
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 3,
    "hidden_size": 192,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "intermediate_size": 512,
    "vocab_size": 384,
    "max_position_embeddings": 256,
    "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_pairing": "neox",
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "tie_word_embeddings": True,
    "attention_bias": False,
    "mlp_bias": False,
    "hidden_act": "silu",
    "bos_token_id": 0,
    "eos_token_id": [3, 5],
}

# A third one whose sizes are no powers of two anywhere, with biases, a head
# size that differs from width / heads, and a rotation of part of each head.
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 4,
    "hidden_size": 120,
    "num_attention_heads": 10,
    "num_key_value_heads": 5,
    "head_dim": 48,
    "rotary_dim": 32,
    "intermediate_size": 264,
    "vocab_size": 1003,
    "max_position_embeddings": 1024,
    "rms_norm_eps": 3e-6,
    "rope_theta": 25000.0,
    "rope_pairing": "neox",
    "rope_scaling": {"rope_type": "linear", "factor": 2.0},
    "tie_word_embeddings": False,
    "attention_bias": True,
    "mlp_bias": True,
    "hidden_act": "silu",
    "bos_token_id": 7,
    "eos_token_id": 11,
}


# A fourth one with the head size of the large models (64) and long enough positions for prompts
# of several hundred tokens: it reaches the kernels that only take that head size.
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2,
    "hidden_size": 96,
    "num_attention_heads": 4,
    "num_key_value_heads": 1,
    "head_dim": 64,
    "intermediate_size": 136,
    "vocab_size": 211,
    "max_position_embeddings": 512,
    "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_pairing": "neox",
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 128},
    "tie_word_embeddings": True,
    "attention_bias": False,
    "mlp_bias": False,
    "hidden_act": "silu",
    "bos_token_id": 1,
    "eos_token_id": 2,
}


# A fifth one with the head size of the larger models (128), three query heads on one KV head (a group
# size that divides nothing), a width that is not heads x head size, and room for prompts of several
# hundred tokens: head size 128 in the decode kernel and in the kernels that only long prompts reach.
TINY_E = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2,
    "hidden_size": 80,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "head_dim": 128,
    "intermediate_size": 104,
    "vocab_size": 173,
    "max_position_embeddings": 512,
    "rms_norm_eps": 2e-6,
    "rope_theta": 10000.0,
    "rope_pairing": "llama",
    "rope_scaling": {"rope_type": "linear", "factor": 4.0},
    "tie_word_embeddings": False,
    "attention_bias": False,
    "mlp_bias": False,
    "hidden_act": "silu",
    "bos_token_id": 3,
    "eos_token_id": 4,
}


def tensor_shapes(cfg: dict) -> dict[str, tuple]:
    """Names and shapes of a checkpoint of this architecture, weights [out, in]."""
    E = cfg["hidden_size"]
    H = cfg["num_attention_heads"]
    K = cfg.get("num_key_value_heads") or H
    D = cfg.get("head_dim") or E // H
    Fi = cfg["intermediate_size"]
    V = cfg["vocab_size"]
    s = {"model.embed_tokens.weight": (V, E)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        s[p + "input_layernorm.weight"] = (E,)
        s[p + "self_attn.q_proj.weight"] = (H * D, E)
        s[p + "self_attn.k_proj.weight"] = (K * D, E)
        s[p + "self_attn.v_proj.weight"] = (K * D, E)
        s[p + "self_attn.o_proj.weight"] = (E, H * D)
        if cfg.get("attention_bias"):
            s[p + "self_attn.q_proj.bias"] = (H * D,)
            s[p + "self_attn.k_proj.bias"] = (K * D,)
            s[p + "self_attn.v_proj.bias"] = (K * D,)
            s[p + "self_attn.o_proj.bias"] = (E,)
        s[p + "post_attention_layernorm.weight"] = (E,)
        s[p + "mlp.gate_proj.weight"] = (Fi, E)
        s[p + "mlp.up_proj.weight"] = (Fi, E)
        s[p + "mlp.down_proj.weight"] = (E, Fi)
        if cfg.get("mlp_bias"):
            s[p + "mlp.gate_proj.bias"] = (Fi,)
            s[p + "mlp.up_proj.bias"] = (Fi,)
            s[p + "mlp.down_proj.bias"] = (E,)
    s["model.norm.weight"] = (E,)
    if not cfg.get("tie_word_embeddings"):
        s["lm_head.weight"] = (V, E)
    return s


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = x + np.uint64(0x9E3779B97F4A7C15)
        z = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def normal(n: int, key: int) -> np.ndarray:
    """n standard normals (float64) from splitmix64 of (key, index) and Box-Muller."""
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64) * np.uint64(2) + (np.uint64(key) << np.uint64(33))
    a = _splitmix64(idx)
    b = _splitmix64(idx + np.uint64(1))
    u1 = ((a >> np.uint64(11)).astype(np.float64) + 1.0) / 9007199254740993.0
    u2 = (b >> np.uint64(11)).astype(np.float64) / 9007199254740992.0
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def make_weights(cfg: dict, seed: int, std: float = 0.02) -> dict[str, np.ndarray]:
    """float32 weights: matrices, biases and embeddings N(0, std); norm weights 1 + N(0, std)."""
    out = {}
    for n, (name, shape) in enumerate(tensor_shapes(cfg).items()):
        v = normal(int(np.prod(shape)), seed * 1000 + n) * std
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            v = 1.0 + v
        out[name] = v.astype(np.float32).reshape(shape)
    return out


def write_safetensors(path, tensors: dict[str, np.ndarray]) -> None:
    """Test-side writer (float32 and int32 only), independent of the package's."""
    header, off, blobs = {}, 0, []
    for name, arr in tensors.items():
        if arr.dtype == np.float32:
            dt = "F32"
        elif arr.dtype == np.int32:
            dt = "I32"
        else:
            raise ValueError(arr.dtype)
        raw = np.ascontiguousarray(arr).astype(arr.dtype.newbyteorder("<")).tobytes()
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def write_model_dir(path, cfg: dict, tensors: dict[str, np.ndarray]) -> Path:
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(path / "model.safetensors", tensors)
    return path


def prompt_tokens(cfg: dict, length: int, seed: int) -> list[int]:
    v = _splitmix64(np.arange(length, dtype=np.uint64) + (np.uint64(seed) << np.uint64(40)))
    return [int(x % np.uint64(cfg["vocab_size"])) for x in v]
