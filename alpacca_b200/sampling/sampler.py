"""Sampling on the device for the rows of a batch.

State per sequence (the reference's `Sampler`, alpacca/sample.py:22-34): the
window of recent tokens (the prompt feeds it, alpacca/chat.py:150-151) and the
number of draws made; the random numbers are keyed by the seed and counted by
(stream, step), a stream being the request's index in the call.
"""
from __future__ import annotations

import torch

from .. import ops
from .params import SamplerParams


class SequenceSamplerState:
    __slots__ = ("stream", "step", "recent", "window")

    def __init__(self, stream: int, prompt, window: int):
        self.stream, self.step, self.window = int(stream), 0, max(int(window), 1)
        self.recent = list(prompt)[-self.window:]

    def accept(self, token: int) -> None:
        self.recent.append(int(token))
        if len(self.recent) > self.window:
            del self.recent[0]


class DeviceSampler:
    def __init__(self, params: SamplerParams, device):
        self.params = params
        self.seed = params.resolved_seed()
        self.device = torch.device(device)

    def new_state(self, stream: int, prompt) -> SequenceSamplerState:
        return SequenceSamplerState(stream, prompt, self.params.repeat_last_n)

    def sample(self, logits: torch.Tensor, states) -> list[int]:
        """Tokens for the rows of `logits` [B,V] (float32, on the device; changed in place by
        the penalty).  Advances each state's step and window."""
        p = self.params
        B = logits.shape[0]
        if p.penalizes and any(s.recent for s in states):
            R = max(len(s.recent) for s in states)
            recent = torch.full((B, R), -1, dtype=torch.int32)
            for b, s in enumerate(states):
                if s.recent:
                    recent[b, :len(s.recent)] = torch.tensor(s.recent, dtype=torch.int32)
            ops.repeat_penalty(logits, recent.to(self.device, non_blocking=True), p.repeat_penalty)
        meta = torch.tensor([[s.stream for s in states], [s.step for s in states]], dtype=torch.int32)
        meta = meta.to(self.device, non_blocking=True)
        out = torch.empty(B, dtype=torch.int32, device=self.device)
        ops.sample(logits, out, p.temperature, p.top_k, p.top_p if 0.0 < p.top_p < 1.0 else 1.0,
                   self.seed, meta[0], meta[1])
        tokens = out.tolist()
        for s, t in zip(states, tokens):
            s.step += 1
            s.accept(t)
        return tokens
