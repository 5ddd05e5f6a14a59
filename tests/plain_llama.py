"""Plain, slow implementation of the Llama-style dense decoder, in NumPy float64.

Whole sequences, no cache, one function for each part.  It shares no code with
the `alpacca_b200` package: it has its own safetensors reader, its own RoPE
tables, its own sampler and its own counter-based random numbers, so that a
fault in the package cannot hide in a shared helper.

Every function is written from the formulas of jtiro232/Alpacca's engine and
cites the file and lines (paths within that project).  The comparison of this
file with the reference's own code, run on the CPU, is
`tests/golden/make_golden.py`; its committed outputs are checked by
`tests/test_plain_vs_golden.py`.

The llama3 frequency scaling, the temperature/top-k/top-p walk in index order
and the Philox generator are not in the reference (it has no RoPE scaling and
uses Python's `random`); those three rest on their published formulas only.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np

F = np.float64


# --------------------------------------------------------------------------
# reading a model folder (own reader: 8-byte little-endian header length,
# JSON header name -> {dtype, shape, data_offsets}, raw little-endian data)
# --------------------------------------------------------------------------

def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_safetensors(path) -> dict[str, np.ndarray]:
    blob = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    data = memoryview(blob)[8 + hlen:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = data[lo:hi]
        dt = info["dtype"]
        if dt == "F32":
            arr = np.frombuffer(buf, dtype="<f4").astype(F)
        elif dt == "BF16":
            arr = _bf16_to_f32(np.frombuffer(buf, dtype="<u2")).astype(F)
        elif dt == "F16":
            arr = np.frombuffer(buf, dtype="<f2").astype(F)
        elif dt == "I32":
            arr = np.frombuffer(buf, dtype="<i4").copy()
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = arr.reshape(info["shape"])
    return out


def read_model_dir(model_dir):
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    return cfg, read_safetensors(model_dir / "model.safetensors")


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embed(table, tokens):
    """x[t,:] = table[token[t],:], no scaling.  alpacca/model.py:482, alpacca/tensor.py:100-113"""
    return np.asarray(table, F)[np.asarray(tokens, np.int64)].copy()


def rmsnorm(x, weight, eps):
    """inv = 1/sqrt(mean(x^2) + eps); y = (x*inv)*w.  alpacca/tensor.py:163-173"""
    x = np.asarray(x, F)
    inv = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return x * inv * np.asarray(weight, F)


def linear(x, w, b=None):
    """y = x @ w.T (+ b), weights stored [out, in].  alpacca/tensor.py:91-97, alpacca/model.py:488-496"""
    y = np.asarray(x, F) @ np.asarray(w, F).T
    if b is not None:
        y = y + np.asarray(b, F)
    return y


def rope_inv_freq(n_rot, theta):
    """inv_freq_i = theta^(-2i/n_rot), i < n_rot/2.  alpacca/model.py:172-176, :389"""
    half = n_rot // 2
    return np.asarray([theta ** (-2.0 * i / n_rot) for i in range(half)], F)


def scale_inv_freq(inv_freq, scaling):
    """Frequency scaling applied once to the table of frequencies.

    Not in the reference (alpacca/model.py:172-176 has the bare frequencies
    only).  llama3: with wavelength lam = 2*pi/f and L the original maximum
    position, f stays if lam < L/high, becomes f/factor if lam > L/low, and is
    blended in between with s = (L/lam - low)/(high - low):
    f' = (1-s)*f/factor + s*f.  linear: f' = f/factor.
    """
    if not scaling:
        return inv_freq
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind in ("default", None):
        return inv_freq
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv_freq / factor
    if kind != "llama3":
        raise ValueError(f"plain: rope scaling {kind}")
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    L = float(scaling["original_max_position_embeddings"])
    out = []
    for f in inv_freq:
        lam = 2.0 * math.pi / f
        if lam < L / high:
            out.append(f)
        elif lam > L / low:
            out.append(f / factor)
        else:
            s = (L / lam - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return np.asarray(out, F)


def rope(x, positions, n_heads, head_dim, n_rot, inv_freq, pairing):
    """Rotate pairs of each head by pos*inv_freq_i; dims >= n_rot pass through.

    pairing "llama": (2i, 2i+1); "neox": (i, n_rot/2+i).
    out_a = x_a*c - x_b*s; out_b = x_a*s + x_b*c.  alpacca/model.py:381-435
    """
    T = len(positions)
    v = np.asarray(x, F).reshape(T, n_heads, head_dim).copy()
    half = n_rot // 2
    theta = np.asarray(positions, F)[:, None] * np.asarray(inv_freq, F)[None, :]
    c = np.cos(theta)[:, None, :]
    s = np.sin(theta)[:, None, :]
    if pairing == "llama":
        a = v[:, :, 0:n_rot:2].copy()
        b = v[:, :, 1:n_rot:2].copy()
        v[:, :, 0:n_rot:2] = a * c - b * s
        v[:, :, 1:n_rot:2] = a * s + b * c
    elif pairing == "neox":
        a = v[:, :, :half].copy()
        b = v[:, :, half:n_rot].copy()
        v[:, :, :half] = a * c - b * s
        v[:, :, half:n_rot] = a * s + b * c
    else:
        raise ValueError(pairing)
    return v


def attention(q, k, v, window=None):
    """Causal grouped-query attention of one whole sequence, per head in a loop.

    q [T,H,D], k,v [T,K,D]; head h reads KV head h // (H/K); score = (q.k) *
    D^-1/2, keys s <= t only, softmax over s, out = sum_s p_s v_s.
    alpacca/model.py:447-467 (grouped form), :581-598 (per-head loop).
    `window` (keys t-window < s <= t) is not in the reference; None = all keys.
    """
    T, H, D = q.shape
    K = k.shape[1]
    G = H // K
    out = np.zeros((T, H, D), F)
    scale = 1.0 / math.sqrt(D)
    for h in range(H):
        kh = k[:, h // G, :]
        vh = v[:, h // G, :]
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            sc = (kh[lo:t + 1] @ q[t, h]) * scale
            sc = sc - sc.max()
            p = np.exp(sc)
            p = p / p.sum()
            out[t, h] = p @ vh[lo:t + 1]
    return out


def swiglu(gate, up):
    """a = gate/(1+exp(-gate)) * up.  alpacca/model.py:513, alpacca/tensor.py:150-160"""
    gate = np.asarray(gate, F)
    return gate / (1.0 + np.exp(-gate)) * np.asarray(up, F)


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------

class PlainLlama:
    """Whole-sequence forward pass from a config.json dict and tensors by name."""

    def __init__(self, cfg: dict, tensors: dict):
        self.cfg = cfg
        self.w = tensors
        self.L = cfg["num_hidden_layers"]
        self.E = cfg["hidden_size"]
        self.H = cfg["num_attention_heads"]
        self.K = cfg.get("num_key_value_heads") or self.H
        self.D = cfg.get("head_dim") or self.E // self.H
        self.eps = cfg.get("rms_norm_eps", 1e-5)
        self.theta = cfg.get("rope_theta", 10000.0)
        self.pairing = cfg.get("rope_pairing", "neox")
        self.n_rot = cfg.get("rotary_dim") or self.D
        self.inv_freq = scale_inv_freq(rope_inv_freq(self.n_rot, self.theta),
                                       cfg.get("rope_scaling"))
        self.tied = bool(cfg.get("tie_word_embeddings", False))

    @classmethod
    def from_dir(cls, model_dir):
        return cls(*read_model_dir(model_dir))

    def _get(self, name):
        return self.w.get(name)

    def block(self, x, i, positions):
        """x += Attn(norm1(x)); x += FFN(norm2(x)).  alpacca/model.py:486-514"""
        p = f"model.layers.{i}."
        w = self.w
        h = rmsnorm(x, w[p + "input_layernorm.weight"], self.eps)
        q = linear(h, w[p + "self_attn.q_proj.weight"], self._get(p + "self_attn.q_proj.bias"))
        k = linear(h, w[p + "self_attn.k_proj.weight"], self._get(p + "self_attn.k_proj.bias"))
        v = linear(h, w[p + "self_attn.v_proj.weight"], self._get(p + "self_attn.v_proj.bias"))
        q = rope(q, positions, self.H, self.D, self.n_rot, self.inv_freq, self.pairing)
        k = rope(k, positions, self.K, self.D, self.n_rot, self.inv_freq, self.pairing)
        v = v.reshape(len(positions), self.K, self.D)
        att = attention(q, k, v).reshape(len(positions), self.H * self.D)
        x = x + linear(att, w[p + "self_attn.o_proj.weight"], self._get(p + "self_attn.o_proj.bias"))
        h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], self.eps)
        g = linear(h, w[p + "mlp.gate_proj.weight"], self._get(p + "mlp.gate_proj.bias"))
        u = linear(h, w[p + "mlp.up_proj.weight"], self._get(p + "mlp.up_proj.bias"))
        x = x + linear(swiglu(g, u), w[p + "mlp.down_proj.weight"], self._get(p + "mlp.down_proj.bias"))
        return x

    def hidden(self, tokens):
        x = embed(self.w["model.embed_tokens.weight"], tokens)
        positions = np.arange(len(tokens))
        for i in range(self.L):
            x = self.block(x, i, positions)
        return x

    def logits(self, tokens):
        """Logits at every position of one whole sequence, [T, V] float64.

        Final norm and head: alpacca/model.py:518 (there the last row only);
        tied head = the embedding table, alpacca/model.py:320-322.
        """
        x = rmsnorm(self.hidden(tokens), self.w["model.norm.weight"], self.eps)
        head = self.w["model.embed_tokens.weight"] if self.tied else self.w["lm_head.weight"]
        return linear(x, head)


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------

_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85
_M32 = 0xFFFFFFFF


def philox4x32(counter, key, rounds=10):
    """Philox-4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3")."""
    c = [x & _M32 for x in counter]
    k = [x & _M32 for x in key]
    for _ in range(rounds):
        p0 = _PHILOX_M0 * c[0]
        p1 = _PHILOX_M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & _M32, p1 & _M32,
             ((p0 >> 32) ^ c[3] ^ k[1]) & _M32, p0 & _M32]
        k = [(k[0] + _PHILOX_W0) & _M32, (k[1] + _PHILOX_W1) & _M32]
    return c


def uniform(seed, stream, step):
    """u in [0,1): the top 24 bits of the first Philox word, key = the 64-bit
    seed, counter = (step, 0, stream, 0)."""
    x = philox4x32([step, 0, stream, 0], [seed & _M32, (seed >> 32) & _M32])[0]
    return (x >> 8) * (1.0 / (1 << 24))


def penalize(logits, recent, penalty):
    """For each distinct recent token: l>0 -> l/p, else l*p.  alpacca/sample.py:40-43"""
    out = np.array(logits, np.float64)
    if penalty and penalty != 1.0:
        for t in set(recent):
            out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out


def sample(logits, temperature, top_k, top_p, u):
    """One token from one row of logits.

    temperature <= 0: first index of the maximum (alpacca/sample.py:45-46,
    alpacca/tensor.py:187-194).  Else keep the top_k largest logits (all if
    top_k <= 0; ties go to the lower index, as Python's stable sort gives,
    alpacca/sample.py:48-51), weights exp((l-max)/T) (:53-54), then the
    shortest prefix in descending order whose probability reaches top_p
    (:58-68).  The reference draws from that list in sorted order with
    Python's `random`; here the kept set is walked in index order and the
    first index whose running sum exceeds u * total is taken.
    """
    l = np.asarray(logits, np.float64)
    if temperature <= 0:
        return int(np.argmax(l))
    order = sorted(range(len(l)), key=lambda i: -l[i])  # stable: ties by index
    k = top_k if top_k and top_k > 0 else len(l)
    order = order[:min(k, len(l))]
    w = np.exp((l[order] - l[order[0]]) / temperature)
    if 0.0 < top_p < 1.0:
        probs = w / w.sum()
        acc, cut = 0.0, len(order)
        for n, pr in enumerate(probs):
            acc += pr
            if acc >= top_p:
                cut = n + 1
                break
        order, w = order[:cut], w[:cut]
    kept = sorted(zip(order, w))
    total = sum(x for _, x in kept)
    target = u * total
    acc = 0.0
    for i, x in kept:
        acc += x
        if acc > target:
            return int(i)
    return int(kept[-1][0])


def generate(model: PlainLlama, prompt, n_predict, temperature=0.0, top_k=0, top_p=1.0,
             repeat_penalty=1.0, repeat_last_n=64, seed=0, stream=0, stop=()):
    """The reference's loop for one sequence, each step from the whole sequence.

    sample -> accept -> count -> stop? -> budget? -> forward.
    alpacca/chat.py:149-178: the prompt feeds the repeat window, a stop token
    is counted but not fed back, the last sampled token is not forwarded.
    Returns (tokens, list of the logits each was sampled from).
    """
    seq = list(prompt)
    recent = list(prompt)[-max(repeat_last_n, 1):]
    out, rows = [], []
    for step in range(n_predict):
        row = model.logits(seq)[-1]
        rows.append(row)
        tok = sample(penalize(row, recent, repeat_penalty), temperature, top_k, top_p,
                     uniform(seed, stream, step))
        out.append(tok)
        recent = (recent + [tok])[-max(repeat_last_n, 1):]
        if tok in stop:
            break
        seq.append(tok)
    return out, rows
