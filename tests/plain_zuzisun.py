"""A plain, slow statement of the Zuzisun decoder, one function per mechanism.

Written from the design's equations in double precision with torch on the CPU; it
shares nothing with the engine (no part, no kernel face, no cache).  A whole
sequence is run at once: the window is a mask, the shifted input is a roll by one
token, nothing is cached.

Notation: ``x`` [n, width] is the residual stream, ``h`` a sublayer's input, ``W``
matrices are stored [out, in] and applied as ``h @ W.T``.
"""
from __future__ import annotations

import json
import math
import os

import torch

F = torch.float64


def read_model_folder(path):
    from inferx_b200.weights.safetensors_io import Checkpoint
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    ck = Checkpoint(path)
    w = {n: ck.get(n).clone() for n in ck.names()}
    ck.close()
    return cfg, w


def round_bf16(t):
    return t.to(torch.float32).to(torch.bfloat16).to(t.dtype)


def round_f32(t):
    return t.to(torch.float32).to(t.dtype)


def same(t):
    return t


# -- mechanisms --------------------------------------------------------------
def grouped_rms_norm(v, gain, groups, eps):
    """Each of ``groups`` equal consecutive parts of a row over its own root mean
    square (eps inside the root); the whole row times ``gain``."""
    n, d = v.shape
    parts = v.reshape(n, groups, d // groups)
    ms = (parts * parts).mean(-1, keepdim=True)
    return (parts / torch.sqrt(ms + eps)).reshape(n, d) * gain


def token_shift(h, mix, before=None):
    """h_t + (h_{t-1} - h_t) * mix, with zeros (or ``before``) ahead of the first row."""
    first = torch.zeros_like(h[:1]) if before is None else before.reshape(1, -1)
    prev = torch.cat([first, h[:-1]], dim=0)
    return h + (prev - h) * mix


def rotary_frequencies(dims, base, scaling=None):
    """(frequency per pair [dims/2], factor on cos and sin)."""
    i = torch.arange(dims // 2, dtype=F)
    f = torch.pow(torch.tensor(float(base), dtype=F), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate_interleaved(v, positions, freq, mag, single=False):
    """v [n, ..., d]: the pairs (2i, 2i+1) for i < len(freq) are turned by
    ``positions * freq[i]``; cos and sin carry the factor ``mag``; the rest passes.
    ``single``: the angle, its cosine and its sine are formed in 32-bit, as an engine
    forms them."""
    r = 2 * freq.numel()
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [freq.numel()]
    if single:
        a = (positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]).reshape(shape)
        c, s = torch.cos(a).to(F) * mag, torch.sin(a).to(F) * mag
    else:
        a = (positions.to(F)[:, None] * freq[None, :]).reshape(shape)
        c, s = torch.cos(a) * mag, torch.sin(a) * mag
    u, w = v[..., 0:r:2], v[..., 1:r:2]
    out = v.clone()
    out[..., 0:r:2] = u * c - w * s
    out[..., 1:r:2] = w * c + u * s
    return out


def window_mask(n, size, offset=0):
    """[n, offset + n] bool: query i (at position offset + i) sees key j iff
    0 <= offset + i - j < size (size 0: every earlier key)."""
    qi = torch.arange(offset, offset + n)[:, None]
    kj = torch.arange(offset + n)[None, :]
    d = qi - kj
    return (d >= 0) & ((d < size) if size > 0 else torch.ones_like(d, dtype=torch.bool))


def latent_attention(h, m, w, prefix, eps, positions, rnd=same, single=False):
    """The latent-attention mixer on its (already shifted) input ``h`` [n, width]."""
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    n = h.shape[0]
    W = lambda name: w[f"{prefix}.{name}"].to(F)
    q = rnd(h @ W("q").T).reshape(n, H, dn + dr)
    down = rnd(h @ W("dkv").T)
    c = down[:, :rank]
    c = rnd(c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * W("dkv.norm"))
    rot = m["rot"]
    freq, mag = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    k_rot = rnd(rotate_interleaved(down[:, None, rank:], positions, freq, mag, single))[:, 0]
    q_rot = rnd(rotate_interleaved(q[..., dn:], positions, freq, mag, single))
    q_plain = q[..., :dn]
    k_plain = rnd(c @ W("uk").T).reshape(n, H, dn)
    v = rnd(c @ W("uv").T).reshape(n, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain)
              + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    size = (m.get("mask") or {}).get("size", 0)
    vis = window_mask(n, size)
    scores = scores.masked_fill(~vis[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    o = rnd(torch.einsum("hij,jhd->ihd", p, v)).reshape(n, H * dv)
    gate = torch.sigmoid(rnd(h @ W("g").T))
    return rnd(rnd(o * gate) @ W("o").T)


def clamped_glu(h, f, w, prefix, rnd=same):
    """min(g, L) * sigmoid(1.702 min(g, L)) * (clamp(u, -L, L) + 1), then down."""
    L = float(f["limit"])
    g = torch.clamp(rnd(h @ w[f"{prefix}.gate"].to(F).T), max=L)
    u = torch.clamp(rnd(h @ w[f"{prefix}.up"].to(F).T), -L, L)
    y = rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0))
    return rnd(y @ w[f"{prefix}.down"].to(F).T)


# -- the model -----------------------------------------------------------------
def forward(cfg, w, tokens, rnd=same, layers_out=None, single_angles=False):
    """Logits [n, vocab] (float64) for one sequence from position 0.  ``rnd`` is
    applied where an engine stores an activation (``round_bf16``, ``round_f32``);
    ``single_angles`` forms the rotation's angles in 32-bit; ``layers_out``, a list,
    receives the residual stream after every layer."""
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    n = ids.numel()
    positions = torch.arange(n)
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"])
    embed = w["embed"].to(F)
    x = embed[ids] * float(cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        if layer["type"] != "latent_attention":
            raise ValueError(f"unknown layer type {layer['type']!r}")
        h = rnd(token_shift(x, w[f"{p}.shift"].to(F)))
        a = latent_attention(h, layer["mixer"], w, f"{p}.mix", eps, positions, rnd,
                             single_angles)
        x = x + grouped_rms_norm(a, w[f"{p}.norm1"].to(F), groups, eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")
            y = clamped_glu(rnd(x), layer["mlp"], w, f"{p}.mlp", rnd)
            x = x + grouped_rms_norm(y, w[f"{p}.norm2"].to(F), groups, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    last = rnd(grouped_rms_norm(x, w["final.norm"].to(F), groups, eps))
    return last @ embed.T
