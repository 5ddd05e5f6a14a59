"""The configuration of the Llama-style dense decoder, by its config.json keys.

The reference reads the same constants from GGUF metadata into `Hyperparams`
(alpacca/model.py:134-148, :195-217); the defaults that it applies are the
defaults here: KV heads = heads (:200), head size = width / heads (:201),
rotated dims = head size (:213), eps 1e-5 (:214), rope base 10000 (:215).
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ModelConfig

ROPE_PAIRINGS = ("llama", "neox")
ROPE_SCALINGS = ("default", "linear", "llama3")


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    num_hidden_layers: int = None            # required (None default is rejected in validate)
    hidden_size: int = None
    num_attention_heads: int = None
    intermediate_size: int = None
    vocab_size: int = None
    num_key_value_heads: int | None = None   # default: num_attention_heads
    head_dim: int | None = None              # default: hidden_size // num_attention_heads
    rotary_dim: int | None = None            # default: head_dim (alpacca/model.py:213)
    max_position_embeddings: int = 4096      # alpacca/model.py:211
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    # "llama": pairs (2i, 2i+1); "neox": pairs (i, half+i).  The reference fixes
    # this per architecture string (alpacca/model.py:22-29).  Checkpoints in the
    # q/k row order of config.json-style folders rotate split halves, so that is
    # the default; it is never guessed from anything else.
    rope_pairing: str = "neox"
    rope_scaling: dict | None = None
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    bos_token_id: int | None = None
    eos_token_id: int | list | None = None
    torch_dtype: str | None = None

    # -- derived sizes -----------------------------------------------------
    @property
    def n_kv_heads(self) -> int:
        return self.num_key_value_heads or self.num_attention_heads

    @property
    def head_size(self) -> int:
        return self.head_dim or self.hidden_size // self.num_attention_heads

    @property
    def n_rot(self) -> int:
        return self.rotary_dim or self.head_size

    @property
    def stop_token_ids(self) -> tuple[int, ...]:
        e = self.eos_token_id
        if e is None:
            return ()
        return tuple(e) if isinstance(e, (list, tuple)) else (int(e),)

    # -- the neutral accessors (config/base.py) ------------------------------------
    @property
    def max_positions(self) -> int:
        return self.max_position_embeddings

    @property
    def bos_token(self) -> int | None:
        return self.bos_token_id

    @property
    def stop_tokens(self) -> tuple[int, ...]:
        return self.stop_token_ids

    def validate(self) -> list[str]:
        bad: list[str] = []
        for name in ("num_hidden_layers", "hidden_size", "num_attention_heads",
                     "intermediate_size", "vocab_size"):
            v = getattr(self, name)
            if v is None:
                bad.append(f"missing key '{name}'")
            elif not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                bad.append(f"key '{name}' must be a positive integer, got {v!r}")
        if bad:
            return bad
        for name in ("num_key_value_heads", "head_dim", "rotary_dim"):
            v = getattr(self, name)
            if v is not None and (not isinstance(v, int) or isinstance(v, bool) or v <= 0):
                bad.append(f"key '{name}' must be a positive integer or absent, got {v!r}")
        if bad:
            return bad
        H, K, D = self.num_attention_heads, self.n_kv_heads, self.head_size
        if self.head_dim is None and self.hidden_size % H:
            bad.append(f"hidden_size {self.hidden_size} is not a multiple of num_attention_heads {H} "
                       "and no head_dim is given")
        if H % K:
            bad.append(f"num_attention_heads {H} is not a multiple of num_key_value_heads {K}")
        if D <= 0:
            bad.append(f"head size {D} must be positive")
        if self.n_rot % 2 or not 0 < self.n_rot <= D:
            bad.append(f"rotary_dim {self.n_rot} must be even and at most the head size {D}")
        if self.max_position_embeddings <= 0:
            bad.append("max_position_embeddings must be positive")
        if not self.rms_norm_eps >= 0:
            bad.append("rms_norm_eps must not be negative")
        if not self.rope_theta > 0:
            bad.append("rope_theta must be positive")
        if self.rope_pairing not in ROPE_PAIRINGS:
            bad.append(f"rope_pairing must be one of {ROPE_PAIRINGS}, got {self.rope_pairing!r}")
        if self.hidden_act != "silu":
            bad.append(f"hidden_act {self.hidden_act!r} is not supported (the feed-forward is SwiGLU: 'silu')")
        rs = self.rope_scaling
        if rs is not None:
            if not isinstance(rs, dict):
                bad.append("rope_scaling must be an object or null")
            else:
                kind = rs.get("rope_type", rs.get("type", "default"))
                if kind not in ROPE_SCALINGS:
                    bad.append(f"rope_scaling type {kind!r} is not supported (supported: {ROPE_SCALINGS})")
                need = {"default": (), "linear": ("factor",),
                        "llama3": ("factor", "low_freq_factor", "high_freq_factor",
                                   "original_max_position_embeddings")}.get(kind, ())
                for k in need:
                    if not isinstance(rs.get(k), (int, float)) or isinstance(rs.get(k), bool):
                        bad.append(f"rope_scaling.{k} must be a number")
                if kind == "llama3" and not bad and rs["high_freq_factor"] == rs["low_freq_factor"]:
                    bad.append("rope_scaling.high_freq_factor must differ from low_freq_factor")
        e = self.eos_token_id
        if e is not None and not isinstance(e, int):
            if not (isinstance(e, (list, tuple)) and all(isinstance(x, int) for x in e)):
                bad.append("eos_token_id must be an integer, a list of integers or null")
        for t in self.stop_token_ids if not bad else ():
            if not 0 <= t < self.vocab_size:
                bad.append(f"eos_token_id {t} lies outside the vocabulary of {self.vocab_size}")
        return bad
