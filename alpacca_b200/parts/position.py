"""Rotary position encoding: the table of angles and how pairs are formed.

inv_freq_i = theta^(-2i/n_rot) for i < n_rot/2 (alpacca/model.py:172-176);
angle = position * inv_freq_i; the tables cos, sin [positions, n_rot/2] are
built once (:352-356).  Pairs (alpacca/model.py:381-435): "llama" (2i, 2i+1),
"neox" (i, n_rot/2 + i); dims >= n_rot pass through.

The reference has no frequency scaling.  Here the frequencies can be rescaled
once before the table is built: "linear" divides them by `factor`; "llama3"
keeps wavelengths shorter than L/high, divides those longer than L/low by
`factor` and blends in between with s = (L/wavelength - low)/(high - low),
L = original_max_position_embeddings.  Angles are formed in float64 and the
tables rounded once to float32, which the rotation kernel reads.
"""
from __future__ import annotations

import math

import torch

from .base import BuildOptions, PositionEncoding

PAIRING_CODES = {"llama": 0, "neox": 1}


def scaled_inv_freq(n_rot: int, theta: float, scaling: dict | None) -> torch.Tensor:
    half = n_rot // 2
    f = torch.tensor([theta ** (-2.0 * i / n_rot) for i in range(half)], dtype=torch.float64)
    if not scaling:
        return f
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind in (None, "default"):
        return f
    factor = float(scaling["factor"])
    if kind == "linear":
        return f / factor
    if kind == "llama3":
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        L = float(scaling["original_max_position_embeddings"])
        lam = 2.0 * math.pi / f
        s = ((L / lam - low) / (high - low)).clamp(0.0, 1.0)   # 1 below L/high, 0 above L/low
        blended = (1.0 - s) * f / factor + s * f
        return torch.where(lam < L / high, f, torch.where(lam > L / low, f / factor, blended))
    raise ValueError(f"rope scaling {kind!r} is not supported")


class RotaryEncoding(PositionEncoding):
    def __init__(self, opts: BuildOptions, head_dim: int, n_rot: int, theta: float, pairing: str,
                 scaling: dict | None = None, max_positions: int | None = None):
        if pairing not in PAIRING_CODES:
            raise ValueError(f"pairing must be one of {tuple(PAIRING_CODES)}, got {pairing!r}")
        if n_rot % 2 or not 0 < n_rot <= head_dim:
            raise ValueError(f"n_rot {n_rot} must be even and at most the head size {head_dim}")
        self.opts = opts
        self.head_dim, self.n_rot, self.theta, self.pairing = int(head_dim), int(n_rot), float(theta), pairing
        self.scaling = dict(scaling) if scaling else None
        self.max_positions = int(max_positions or opts.max_positions)
        inv = scaled_inv_freq(self.n_rot, self.theta, self.scaling)
        ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos = torch.cos(ang).to(torch.float32).to(opts.device).contiguous()
        self.sin = torch.sin(ang).to(torch.float32).to(opts.device).contiguous()

    def rotation(self):
        return self.cos, self.sin, self.n_rot, PAIRING_CODES[self.pairing]
