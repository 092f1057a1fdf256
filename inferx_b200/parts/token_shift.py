"""Token shift: what a mixer reads is blended with the previous token's.

``h_t <- h_t + (h_{t-1} - h_t) * mix`` per channel, where ``h_{t-1}`` is the previous
token's value before its own replacement and zeros stand before a sequence's first
token.  The last row a sequence brought is per-request state (fp32, one row of the
model's width per layer), so that the next step - a further portion of the prompt or
a decoded token - continues where this one ended; a request's slot is zeroed when it
is handed out, which gives the zeros before position 0.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import StateNeed
from .registry import register_part

STATE_NAME = "shift_prev"


class TokenShift:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.name = spec, ctx, prefix
        self.mix = None

    def tensors(self):
        return [TensorDecl(self.name, (self.spec.size,), keep="float32", init="bias")]

    def bind(self, weights):
        self.mix = weights[self.name]

    def cache_needs(self):
        return [StateNeed(STATE_NAME, (self.spec.size,), torch.float32)]

    def forward(self, resid, step, cache):
        """The shifted rows in the run's element type; updates the state."""
        return self.ctx.ops.token_shift(resid, self.mix, cache.state[STATE_NAME], step,
                                        self.ctx.dtype)


register_part("mixer_input", "token_shift", TokenShift)
