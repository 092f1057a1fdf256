"""Mixers that carry a matrix of state per head instead of a record per token.

Both kinds here keep ``S [heads, dim, vdim]`` in fp32 per request (a state slot of the
cache manager, zeroed when the slot is handed out) and walk a sequence's tokens in
order with a decay per key channel:

* gated linear attention:  S_t = diag(a_t) S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t
* wkv time mixing:         o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t;
                           S_t = diag(w_t) S_(t-1) + k_t v_t^T

The recurrence, the decays (sigmoid, logarithms, exponentials), the per-head norm of
the output and the gate's silu are fp32; the projections are the run's matrix products.
One kernel serves both recurrences (``ops.linear_recurrence``): a sequence's state
column is owned by one thread from its first token of the step to its last, so a
position's result does not depend on how the sequence was cut into steps or on what
else is in the batch; long prompt portions are cut into segments that are walked side by
side and joined, which changes results by rounding only.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import StateNeed
from .registry import register_part

STATE = "recurrent_state"
PREVIOUS = "previous_input"


def _rank(spec_rank: int) -> int:
    """A declared inner size; -1 (any) when the spec leaves it to the checkpoint."""
    return spec_rank if spec_rank > 0 else -1


class GatedLinearAttention:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.p = spec, ctx, prefix
        self.front_w = self.a2_w = self.a2_b = self.norm_w = self.o_w = None

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_recurrence_limits", None)
        if check is not None:
            check(self.spec.dim, self.p)

    def tensors(self):
        s, p = self.spec, self.p
        hk, hv, r = s.heads * s.dim, s.heads * s.vdim, _rank(s.decay_rank)
        return [
            TensorDecl(f"{p}.q", (hk, s.hidden)), TensorDecl(f"{p}.k", (hk, s.hidden)),
            TensorDecl(f"{p}.v", (hv, s.hidden)), TensorDecl(f"{p}.g", (hv, s.hidden)),
            TensorDecl(f"{p}.o", (s.hidden, hv)),
            TensorDecl(f"{p}.norm", (s.vdim,), keep="float32", init="gain"),
            TensorDecl(f"{p}.a1", (r, s.hidden)),
            TensorDecl(f"{p}.a2", (hk, r), keep="float32"),
            TensorDecl(f"{p}.a2.b", (hk,), keep="float32", init="bias"),
        ]

    def bind(self, w):
        p = self.p
        if w[f"{p}.a1"].shape[0] != w[f"{p}.a2"].shape[1]:
            raise ValueError(f"{p}: a1 has {w[f'{p}.a1'].shape[0]} rows, a2 "
                             f"{w[f'{p}.a2'].shape[1]} columns")
        # one product for everything that reads h: q | k | v | g | a1
        self.front_w = torch.cat([w[f"{p}.q"], w[f"{p}.k"], w[f"{p}.v"], w[f"{p}.g"],
                                  w[f"{p}.a1"]], dim=0).contiguous()
        self.rank = w[f"{p}.a1"].shape[0]
        self.a2_t, self.a2_b = w[f"{p}.a2"].t().contiguous(), w[f"{p}.a2.b"]
        self.norm_w, self.o_w = w[f"{p}.norm"], w[f"{p}.o"]

    def cache_needs(self):
        s = self.spec
        return [StateNeed(STATE, (s.heads, s.dim, s.vdim), torch.float32)]

    def forward(self, x, step, cache):
        s, ops = self.spec, self.ctx.ops
        hk, hv = s.heads * s.dim, s.heads * s.vdim
        front = ops.linear(x, self.front_w)                  # [T, 2 hk + 2 hv + rank]
        q, k, v = front[:, :hk], front[:, hk:2 * hk], front[:, 2 * hk:2 * hk + hv]
        gate, low = front[:, 2 * hk + hv:2 * hk + 2 * hv], front[:, 2 * hk + 2 * hv:]
        decay = ops.lowrank_decay(low, self.a2_t, self.a2_b, mode="sigmoid_root",
                                  tau=s.tau)                             # fp32 [T, hk]
        o = ops.linear_recurrence(q, k, v, decay, None, cache.state[STATE], step, s.heads,
                                  s.dim, s.vdim, q_scale=s.q_scale,
                                  bonus_form=False)                      # fp32 [T, heads, vdim]
        y = ops.head_norm_gate(o, self.norm_w, gate, s.norm_eps, self.ctx.dtype)
        return ops.linear(y, self.o_w, out_dtype=torch.float32)


class WkvMixer:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.p = spec, ctx, prefix

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_recurrence_limits", None)
        if check is not None:
            check(self.spec.dim, self.p)

    def tensors(self):
        s, p = self.spec, self.p
        hk, r = s.heads * s.dim, _rank(s.decay_rank)
        decls = [TensorDecl(f"{p}.mu.{n}", (s.hidden,), keep="float32", init="bias")
                 for n in ("r", "k", "v", "g", "w")]
        decls += [TensorDecl(f"{p}.{n}", (hk, s.hidden)) for n in ("r", "k", "v", "g")]
        decls += [
            TensorDecl(f"{p}.w1", (r, s.hidden)),
            TensorDecl(f"{p}.w2", (hk, r), keep="float32"),
            TensorDecl(f"{p}.w0", (hk,), keep="float32", init="bias"),
            TensorDecl(f"{p}.u", (s.heads, s.dim), keep="float32", init="bias"),
            TensorDecl(f"{p}.norm", (hk,), keep="float32", init="gain"),
            TensorDecl(f"{p}.o", (s.hidden, hk)),
        ]
        return decls

    def bind(self, w):
        p = self.p
        if w[f"{p}.w1"].shape[0] != w[f"{p}.w2"].shape[1]:
            raise ValueError(f"{p}: w1 has {w[f'{p}.w1'].shape[0]} rows, w2 "
                             f"{w[f'{p}.w2'].shape[1]} columns")
        self.mu = torch.stack([w[f"{p}.mu.{n}"] for n in ("r", "k", "v", "g", "w")]).contiguous()
        self.rkvg_w = torch.stack([w[f"{p}.{n}"] for n in ("r", "k", "v", "g")]).contiguous()
        self.w1 = w[f"{p}.w1"]
        self.rank = self.w1.shape[0]
        self.w2_t, self.w0 = w[f"{p}.w2"].t().contiguous(), w[f"{p}.w0"]
        self.u = w[f"{p}.u"].contiguous()
        self.norm_w, self.o_w = w[f"{p}.norm"], w[f"{p}.o"]

    def cache_needs(self):
        s = self.spec
        return [StateNeed(STATE, (s.heads, s.dim, s.dim), torch.float32),
                StateNeed(PREVIOUS, (s.hidden,), torch.float32)]

    def forward(self, x, step, cache):
        s, ops = self.spec, self.ctx.ops
        mixes = ops.shift_mix(x, self.mu, cache.state[PREVIOUS], step)      # [5, T, hidden]
        rkvg = ops.batched_linear(mixes[:4], self.rkvg_w)                    # [4, T, hk]
        lora = ops.linear(mixes[4], self.w1, out_dtype=torch.float32)                               # [T, rank]
        decay = ops.lowrank_decay(lora, self.w2_t, self.w0, mode="exp_exp_tanh")
        o = ops.linear_recurrence(rkvg[0], rkvg[1], rkvg[2], decay, self.u, cache.state[STATE],
                                  step, s.heads, s.dim, s.dim, q_scale=1.0, bonus_form=True)
        y = ops.head_norm_gate(o, self.norm_w, rkvg[3], s.norm_eps, self.ctx.dtype)
        return ops.linear(y, self.o_w, out_dtype=torch.float32)


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "wkv", WkvMixer)
