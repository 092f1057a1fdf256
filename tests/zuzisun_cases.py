"""Shared pieces of the Zuzisun tests: small configurations, model folders, the plain
model's rows and the error bounds."""
import random

import torch

import plain_zuzisun as plain
from inferx_b200.weights.random_model import write_random_model


def latent_layer(heads, dim, rot_dim, vdim, kv_rank, scale, window=0, rot_dims=None, base=10000.0,
                 scaling=None, ff=0, limit=1.0):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
             "scale": scale,
             "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if scaling:
        mixer["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window:
        mixer["mask"] = {"size": window}
    mlp = {"kind": "dense", "ff": ff, "limit": limit} if ff else None
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


# three norm groups, a layer without feed-forward, fewer turned entries than rot_dim,
# value size unlike the key size, windows that differ between layers
ZA = {
    "architecture": "Zuzisun", "vocab": 200, "width": 96, "embedding": {"scale": 2.0},
    "norm": {"eps": 1e-6, "groups": 3},
    "layers": [
        latent_layer(3, 24, 16, 20, 40, 0.21, window=10, scaling=(8.0, 64, 16.0, 2.0), ff=112,
                     limit=0.8),
        latent_layer(3, 24, 16, 20, 40, 0.21, window=7, rot_dims=8),
        latent_layer(2, 8, 24, 36, 24, 0.3, window=10, base=500.0, ff=40, limit=2.5),
    ],
}

# one norm group, no embedding scale, a layer that sees every earlier token, odd head count
ZB = {
    "architecture": "Zuzisun", "vocab": 384, "width": 128, "embedding": {"scale": 1.0},
    "norm": {"eps": 1e-5, "groups": 1},
    "layers": [
        latent_layer(5, 16, 8, 32, 48, 0.25, window=33, scaling=(2.0, 32, 8.0, 1.0), ff=192,
                     limit=1.2),
        latent_layer(5, 16, 8, 32, 48, 0.25, base=100000.0, ff=64, limit=0.5),
        latent_layer(4, 32, 32, 16, 72, 0.15, window=64, scaling=(16.0, 128, 32.0, 0.5), ff=192,
                     limit=7.0),
    ],
}

# sizes of the kind the tensor-core paths take, two layers
ZC = {
    "architecture": "Zuzisun", "vocab": 512, "width": 512, "embedding": {"scale": 1.5},
    "norm": {"eps": 1e-5, "groups": 8},
    "layers": [
        latent_layer(16, 48, 32, 80, 256, 0.1, window=100, scaling=(6.0, 256, 16.0, 2.0), ff=1024,
                     limit=2.0),
        latent_layer(16, 48, 32, 80, 256, 0.1, window=48, scaling=(6.0, 256, 16.0, 2.0), ff=1024,
                     limit=2.0),
    ],
}


# nothing a multiple of 8, an odd vocabulary, one head, a window of one page and of two tokens
ZD = {
    "architecture": "Zuzisun", "vocab": 101, "width": 60, "embedding": {"scale": 0.7},
    "norm": {"eps": 1e-5, "groups": 5},
    "layers": [
        latent_layer(3, 10, 6, 14, 22, 0.3, window=4, rot_dims=4, scaling=(3.0, 16, 4.0, 0.5), ff=50,
                     limit=1.0),
        latent_layer(1, 18, 2, 9, 13, 0.4, window=2, base=50.0, ff=26, limit=3.0),
        latent_layer(7, 4, 10, 6, 30, 0.5, rot_dims=0),
    ],
}


# one layer for each latent size the tensor-core attention is built for, beside ZC's 256
ZE = {
    "architecture": "Zuzisun", "vocab": 300, "width": 192, "embedding": {"scale": 1.25},
    "norm": {"eps": 1e-5, "groups": 2},
    "layers": [
        latent_layer(4, 32, 64, 32, 512, 0.12, window=70, scaling=(2.0, 64, 8.0, 1.0), ff=256,
                     limit=1.5),
        latent_layer(6, 40, 16, 24, 128, 0.2, base=1000.0, ff=128, limit=4.0),
        latent_layer(2, 16, 48, 56, 64, 0.25, window=33, rot_dims=32),
    ],
}


def sharpen(name, t):
    """N(0, 0.02) weights would give uniform attention, a dead gate, clamps that never
    act and a shift of nothing; make each of them matter."""
    if name == "embed":
        return t * 40.0
    if name.endswith(".shift"):
        return (t * 25.0).clamp(-0.2, 1.2)          # mostly between 0 and 1
    if name.endswith((".mix.q", ".mix.uk")):
        return t * 8.0
    if name.endswith((".mix.dkv", ".mix.g")):
        return t * 4.0
    if name.endswith((".mlp.gate", ".mlp.up")):
        return t * 6.0
    return t


def sharpen_mildly(name, t):
    """For wide latents, where ``sharpen``'s factors turn attention into an argmax that
    rounding flips: scores with a spread of a few units."""
    if name.endswith((".mix.q", ".mix.uk")):
        return t * 2.5
    return sharpen(name, t)


def make_model_dir(cfg, path, seed, dtype="float32", adjust=None):
    if adjust is None:
        wide = max(l["mixer"]["kv_rank"] for l in cfg["layers"]) >= 256
        adjust = sharpen_mildly if wide else sharpen
    write_random_model(cfg, str(path), seed=seed, dtype=dtype, adjust=adjust)
    return str(path)


def make_requests(cfg, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)]
            for i, n in enumerate(lengths)}


def reference_rows(model_dir, requests):
    cfg, w = plain.read_model_folder(model_dir)
    rows = {}
    for rid, toks in requests.items():
        lg = plain.forward(cfg, w, toks).to(torch.float32)
        for p in range(len(toks)):
            rows[(rid, p)] = lg[p]
    return rows


def bf16_bound(model_dir, requests, factor=3.0, floor=5e-3):
    """``factor`` times what rounding every stored activation to bfloat16 costs the plain
    model itself, relative to the largest logit."""
    cfg, w = plain.read_model_folder(model_dir)
    worst = 0.0
    for toks in requests.values():
        a = plain.forward(cfg, w, toks)
        b = plain.forward(cfg, w, toks, plain.round_bf16)
        worst = max(worst, float((a - b).abs().max()) / float(a.abs().max()))
    return max(floor, factor * worst)


def f32_bound(model_dir, requests, factor=3.0, floor=3e-5):
    """The same for a 32-bit engine: activations stored in 32-bit and the rotation's angle,
    cosine and sine formed in 32-bit (at position p and frequency f the angle alone is off
    by up to p * f * 2^-24 radians, which a sharp score multiplies).  The floor stands for
    what the plain model does not have: sums of hundreds of 32-bit products."""
    cfg, w = plain.read_model_folder(model_dir)
    worst = 0.0
    for toks in requests.values():
        a = plain.forward(cfg, w, toks)
        b = plain.forward(cfg, w, toks, plain.round_f32, single_angles=True)
        worst = max(worst, float((a - b).abs().max()) / float(a.abs().max()))
    return max(floor, factor * worst)


def bound_for(dtype, model_dir, requests):
    return f32_bound(model_dir, requests) if dtype == "float32" else bf16_bound(model_dir, requests)
