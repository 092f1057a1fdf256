"""The Tinapel design stated once more, slowly and in float64, one function per mechanism.

Nothing here is shared with the engine: no kernel, no part, no cache.  A model is a
parsed config.json (a dict) and a dict of tensors by checkpoint name; ``forward`` runs
one whole sequence from position 0 and returns the logits of every position (and, when
asked, the residual stream after every layer run).

Notation: ``h`` is a mixer's or feed-forward's input (a normed row of the stream ``x``),
``H`` heads, ``K`` key entries per head, ``V`` value entries per head.
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


def same(t):
    return t


def round_bf16(t):
    return t.to(torch.float32).to(torch.bfloat16).to(t.dtype)


def round_f32(t):
    return t.to(torch.float32).to(t.dtype)


# What a run in a narrower element type stores between its kernels passes through
# ``_store`` (the identity for the exact model; ``forward(..., store=round_bf16)`` imitates
# a bfloat16 run to measure what its rounding alone costs).
_store = same


def st(t):
    return _store(t)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def sinusoid(positions, width):
    """Entry 2i: sin(p * 10000^(-2i/width)); entry 2i+1: cos of the same angle."""
    out = torch.zeros(len(positions), width, dtype=F)
    p = torch.as_tensor(positions, dtype=F)[:, None]
    for i in range((width + 1) // 2):
        a = p[:, 0] * 10000.0 ** (-2.0 * i / width)
        out[:, 2 * i] = torch.sin(a)
        if 2 * i + 1 < width:
            out[:, 2 * i + 1] = torch.cos(a)
    return out


def embedding(w, cfg, tokens):
    x = w["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    return x + sinusoid(list(range(len(tokens))), cfg["width"])


# ---------------------------------------------------------------------------------------
def gla_mixer(w, p, m, h, eps):
    """Gated linear attention with a decay per key channel.
    S_t = diag(a_t) S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t."""
    T = h.shape[0]
    H, K = m["heads"], m["dim"]
    V = m.get("vdim", K)
    g = lambda n: w[f"{p}.{n}"].to(F)
    q = st(h @ g("q").T).view(T, H, K) * K ** -0.5
    k = st(h @ g("k").T).view(T, H, K)
    v = st(h @ g("v").T).view(T, H, V)
    z = st(h @ g("a1").T) @ g("a2").T + g("a2.b")
    a = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, K)
    S = torch.zeros(H, K, V, dtype=F)
    o = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms(o, eps) * g("norm")
    return st(o.reshape(T, H * V) * silu(st(h @ g("g").T))) @ g("o").T


def attention_mixer(w, p, m, h, eps):
    """Softmax attention whose values are its keys as projected (before the key norm),
    with query/key RMS norm, a query temperature that grows with the position, and
    scores squashed by tanh."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    g = lambda n: w[f"{p}.{n}"].to(F)
    q = st(h @ g("q").T).view(T, H, D)
    k_raw = st(h @ g("k").T).view(T, G, D)
    v = k_raw
    q = rms(q, eps) * g("q.norm")
    k = st(rms(k_raw, eps) * g("k.norm"))
    qt = m.get("q_temp")
    if qt:
        pos = torch.arange(T, dtype=F)
        q = q * (1.0 + qt["coef"] * torch.log(torch.floor((pos + 1) / qt["every"]) + 1.0))[:, None, None]
    q = st(q)
    out = torch.zeros(T, H, D, dtype=F)
    cap = m.get("softcap")
    for hh in range(H):
        kv = hh // (H // G)
        s = (q[:, hh] @ k[:, kv].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
        out[:, hh] = torch.softmax(s, -1) @ v[:, kv]
    return st(out.reshape(T, H * D)) @ g("o").T


def wkv_mixer(w, p, m, h, eps):
    """Time mixing with a per-channel decay and a bonus for the current token.
    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t;  S_t = diag(w_t) S_(t-1) + k_t v_t^T."""
    T = h.shape[0]
    H, K = m["heads"], m["dim"]
    g = lambda n: w[f"{p}.{n}"].to(F)
    prev = torch.cat([torch.zeros(1, h.shape[1], dtype=F), h[:-1]], 0)
    mix = lambda s: st(h + (prev - h) * g(f"mu.{s}"))
    r = st(mix("r") @ g("r").T).view(T, H, K)
    k = st(mix("k") @ g("k").T).view(T, H, K)
    v = st(mix("v") @ g("v").T).view(T, H, K)
    gate = silu(st(mix("g") @ g("g").T))
    dec = torch.exp(-torch.exp(torch.tanh(mix("w") @ g("w1").T) @ g("w2").T + g("w0"))).view(T, H, K)
    u = g("u").view(H, K)
    S = torch.zeros(H, K, K, dtype=F)
    o = torch.zeros(T, H, K, dtype=F)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = dec[t][:, :, None] * S + kv
    o = rms(o, eps).reshape(T, H * K) * g("norm")
    return st(o * gate) @ g("o").T


MIXERS = {"gla": gla_mixer, "attention": attention_mixer, "wkv": wkv_mixer}


# ---------------------------------------------------------------------------------------
def expert(w, p, h):
    g = lambda n: w[f"{p}.{n}"].to(F)
    return st(st(silu(h @ g("gate").T) * (h @ g("up").T)) @ g("down").T)


def route(w, p, mlp, h):
    """(chosen experts [T, top], their weights [T, top])."""
    r = mlp["router"]
    s = torch.softmax(h @ w[f"{p}.router"].to(F).T, -1)
    top_s, top_i = torch.topk(s, r["top"], dim=-1)
    return top_i, top_s / (top_s.sum(-1, keepdim=True) + 1e-20) * r["scale"]


def moe(w, p, mlp, h):
    top_i, top_w = route(w, p, mlp, h)
    out = torch.zeros(h.shape[0], w[f"{p}.e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e, c in zip(top_i[t].tolist(), top_w[t]):
            out[t] += c * expert(w, f"{p}.e{e}", h[t:t + 1])[0]
    if mlp.get("shared"):
        out = out + expert(w, f"{p}.shared", h)
    return st(out)


# ---------------------------------------------------------------------------------------
def layer(w, cfg, i, x):
    lc, eps = cfg["layers"][i], cfg["norm"]["eps"]
    d = MIXERS[lc["type"]](w, f"l{i}.mix", lc["mixer"],
                           st(norm_one_plus(x, w[f"l{i}.norm1"].to(F), eps)), eps)
    if lc.get("mlp") is not None:
        d = d + moe(w, f"l{i}.mlp", lc["mlp"], st(norm_one_plus(x, w[f"l{i}.norm2"].to(F), eps)))
    return x + d


def layer_runs(cfg):
    """[(layer, pass or None)] in the order they run; the pass is given at the first layer
    of each pass through the repeated stretch."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(w, cfg, tokens, want_stream=False, store=same):
    global _store
    _store = store
    try:
        return _forward(w, cfg, tokens, want_stream)
    finally:
        _store = same


def _forward(w, cfg, tokens, want_stream):
    x0 = embedding(w, cfg, tokens)
    x = x0.clone()
    stream = []
    for i, t in layer_runs(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"].to(F)[t]
        x = layer(w, cfg, i, x)
        stream.append(x.clone())
    n = st(norm_one_plus(x, w["final.norm"].to(F), cfg["norm"]["eps"]))
    logits = n @ w["embed"].to(F).T
    return (logits, torch.stack(stream)) if want_stream else logits
