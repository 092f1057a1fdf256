"""Latent attention: keys and values of all heads are widened from one small cached
vector per token.

Per token the input is projected down to ``kv_rank + rot_dim`` numbers: the first
``kv_rank``, RMS-normed, are the latent ``c``; the rest is a rotated key part shared by
all heads.  Head h's key is ``(W_uk[h] c | k_rot)`` and its value ``W_uv[h] c``; only
``c`` and ``k_rot`` are cached, as one record per token.  The key matrix is folded into
the query instead of widening cached latents:

    q_plain . (W_uk[h] c) = (W_uk[h]^T q_plain) . c

so attention runs with one shared key head of ``kv_rank + rot_dim`` entries whose values
are the latents themselves, and the head's output ``sum_j p_j c_j`` is widened by
``W_uv[h]`` afterwards.  Every step - a whole prompt, a portion, a decoded token - takes
this one path through the cache, so a position's result does not depend on how its
sequence was cut.  Queries carry ``dim`` plain and ``rot_dim`` rotated entries per head;
an optional sigmoid gate computed from the mixer's input multiplies the heads' outputs
before the output projection.

The projections that read the input (query, down-projection, gate) are one product over
concatenated weights; the per-head products are library calls batched over heads.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import PagedKvNeed
from .registry import build_part, register_part

ENTRY = "latent"


class LatentAttentionMixer:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        self.position = build_part("position", spec.position, ctx, prefix)
        self.names = dict(spec.names)
        self.in_w = self.uk_t = self.uv = self.o_w = self.latent_gain = None
        s = spec
        self.q_width = s.heads * (s.dim + s.rot_dim)
        self.kv_off = self.q_width
        self.gate_off = self.q_width + s.kv_rank + s.rot_dim

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_latent_attention_limits", None)
        if check is not None:
            check(self.spec.kv_rank, self.spec.rot_dim, self.prefix)

    def _n(self, key):
        return f"{self.prefix}.{self.names[key]}"

    def tensors(self):
        s = self.spec
        hv = s.heads * s.vdim
        decls = [
            TensorDecl(self._n("q"), (self.q_width, s.hidden)),
            TensorDecl(self._n("dkv"), (s.kv_rank + s.rot_dim, s.hidden)),
            TensorDecl(self._n("dkv_norm"), (s.kv_rank,), keep="float32", init="gain"),
            TensorDecl(self._n("uk"), (s.heads * s.dim, s.kv_rank)),
            TensorDecl(self._n("uv"), (hv, s.kv_rank)),
            TensorDecl(self._n("o"), (s.hidden, hv)),
        ]
        if s.output_gate:
            decls.append(TensorDecl(self._n("g"), (hv, s.hidden)))
        return decls

    def bind(self, w):
        s = self.spec
        parts = [w[self._n("q")], w[self._n("dkv")]]
        if s.output_gate:
            parts.append(w[self._n("g")])
        self.in_w = torch.cat(parts, dim=0).contiguous()
        self.latent_gain = w[self._n("dkv_norm")]
        # [heads, kv_rank, dim]: q_lat[h] = q_plain[h] . uk[h] summed over dim
        self.uk_t = w[self._n("uk")].view(s.heads, s.dim, s.kv_rank).transpose(1, 2).contiguous()
        self.uv = w[self._n("uv")].view(s.heads, s.vdim, s.kv_rank).contiguous()
        self.o_w = w[self._n("o")]

    def cache_needs(self):
        s = self.spec
        return [PagedKvNeed(1, s.kv_rank + s.rot_dim, s.window, entries=(ENTRY,))]

    def forward(self, x, step, cache):
        s, ops = self.spec, self.ctx.ops
        T = x.shape[0]
        group = step.groups[cache.group]
        records = cache.pages[ENTRY]
        proj = ops.linear(x, self.in_w)
        if self.position is not None:
            freq, mag, rot_dims = self.position.pair_table()
        else:
            freq, mag, rot_dims = torch.empty(0, dtype=torch.float32, device=x.device), 1.0, 0
        q_rot, q_plain = ops.latent_prepare(
            proj, 0, self.kv_off, step.positions, freq, mag, self.latent_gain, s.latent_eps,
            s.heads, s.dim, s.rot_dim, rot_dims, s.kv_rank,
            records if cache.writes else None, group.slots if cache.writes else None)
        q_lat = ops.batched_linear(q_plain, self.uk_t)                       # [heads, T, rank]
        mixed = ops.latent_attention(q_lat, q_rot, records, group.block_table, step, s.window,
                                     s.scale)                                # [heads, T, rank]
        o = ops.batched_linear(mixed, self.uv)                               # [heads, T, vdim]
        if s.output_gate:
            o = ops.gate_heads(o, proj, self.gate_off)
        else:
            o = o.transpose(0, 1).reshape(T, s.heads * s.vdim)
        return ops.linear(o, self.o_w, out_dtype=torch.float32)


register_part("mixer", "latent_attention", LatentAttentionMixer)
