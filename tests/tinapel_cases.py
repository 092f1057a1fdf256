"""Shared pieces of the Tinapel tests: small configurations, model folders, the plain
model's rows and the error bounds."""
import random

import torch

import plain_tinapel as plain
from inferx_b200.weights.random_model import write_random_model


def moe(experts, top, ff, scale=1.0, shared=0):
    out = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def wkv(heads, dim, rank, mlp=None):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "rank": rank}, "mlp": mlp}


def gla(heads, dim, vdim, tau, rank, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau,
                                     "rank": rank}, "mlp": mlp}


def attention(heads, kv_heads, dim, scale, softcap=0.0, q_temp=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if softcap:
        m["softcap"] = softcap
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


# the first two layers run three times; a layer without feed-forward; value size unlike the
# key size; a temperature that changes every 4 positions; scores squashed hard
TA = {
    "architecture": "Tinapel", "vocab": 200, "width": 96, "embedding": {"scale": 3.0},
    "norm": {"eps": 1e-6},
    "layers": [
        gla(3, 8, 12, 4.0, 5, moe(4, 2, 24, 1.0, shared=40)),
        attention(4, 2, 20, 0.3, softcap=4.0, q_temp=(0.5, 4)),
        wkv(2, 16, 6, moe(5, 1, 32, 2.5)),
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
}

# no loop, no embedding scale, as many key/value heads as heads, no squashing and no
# temperature, every expert chosen, no shared expert, one head
TB = {
    "architecture": "Tinapel", "vocab": 384, "width": 128, "embedding": {"scale": 1.0},
    "norm": {"eps": 1e-5},
    "layers": [
        wkv(4, 32, 8, moe(3, 3, 48, 0.5)),
        attention(2, 2, 36, 0.2, mlp=moe(6, 2, 40, 1.0, shared=16)),
        gla(1, 40, 24, 9.0, 12, moe(2, 1, 64, 1.0, shared=64)),
        wkv(1, 24, 3),
    ],
}

# nothing a multiple of 8, odd head sizes, an odd vocabulary; one layer repeated
TC = {
    "architecture": "Tinapel", "vocab": 101, "width": 60, "embedding": {"scale": 0.7},
    "norm": {"eps": 1e-5},
    "layers": [
        attention(3, 1, 9, 0.45, softcap=30.0, q_temp=(0.2, 7), mlp=moe(3, 2, 26, 1.5, shared=10)),
        wkv(5, 7, 4, moe(3, 2, 26, 1.5, shared=10)),
        gla(4, 3, 5, 2.0, 2, moe(7, 3, 18, 1.0)),
    ],
    "loop": {"start": 1, "stop": 2, "times": 2},
}

# sizes of the kind the tensor-core paths take; the whole model runs twice
TD = {
    "architecture": "Tinapel", "vocab": 512, "width": 256, "embedding": {"scale": 16.0},
    "norm": {"eps": 1e-5},
    "layers": [
        wkv(4, 64, 32, moe(8, 2, 128, 1.0, shared=128)),
        gla(2, 64, 128, 12.0, 24, moe(8, 2, 128, 1.0, shared=128)),
        attention(8, 2, 64, 0.125, softcap=20.0, q_temp=(0.25, 32), mlp=moe(8, 2, 128, 2.0, shared=256)),
        attention(4, 1, 128, 0.09, q_temp=(0.1, 10), mlp=moe(4, 4, 64, 1.0)),
    ],
    "loop": {"start": 0, "stop": 4, "times": 2},
}

CONFIGS = {"TA": TA, "TB": TB, "TC": TC, "TD": TD}


def sharpen(name, t):
    """N(0, 0.02) weights would give uniform attention, decays that never differ, a dead
    gate, a router without preferences and a shift of nothing; make each of them matter."""
    if name == "embed":
        return t * 40.0
    if ".mix.mu." in name:
        return (t * 25.0).clamp(-0.2, 1.2)
    if name.endswith((".mix.q", ".mix.k", ".mix.r")):
        return t * 6.0
    if name.endswith((".mix.v", ".mix.g")):
        return t * 4.0
    if name.endswith((".mix.w1", ".mix.a1")):
        return t * 10.0
    if name.endswith((".mix.w2", ".mix.a2")):
        return t * 30.0
    if name.endswith(".mix.w0"):
        return t * 50.0 - 1.0            # decays spread around exp(-exp(-1))
    if name.endswith(".mix.a2.b"):
        return t * 50.0 + 2.0
    if name.endswith(".mix.u"):
        return t * 25.0
    if name.endswith(".router"):
        return t * 12.0
    if name.endswith((".gate", ".up")):
        return t * 6.0
    if name == "loop.step":
        return t * 20.0
    return t


def make_model_dir(cfg, path, seed, dtype="float32", adjust=sharpen):
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
        lg = plain.forward(w, cfg, toks).to(torch.float32)
        for p in range(len(toks)):
            rows[(rid, p)] = lg[p]
    return rows


def _bound(model_dir, requests, store, factor, floor):
    cfg, w = plain.read_model_folder(model_dir)
    worst = 0.0
    for toks in requests.values():
        a = plain.forward(w, cfg, toks)
        b = plain.forward(w, cfg, toks, store=store)
        worst = max(worst, float((a - b).abs().max()) / float(a.abs().max()))
    return max(floor, factor * worst)


def bound_for(dtype, model_dir, requests):
    """Three times what storing activations in the run's element type costs the plain
    model itself, relative to the largest logit; the floors stand for sums of hundreds of
    products in that precision, which the plain model does not have."""
    if dtype == "float32":
        return _bound(model_dir, requests, plain.round_f32, 3.0, 3e-5)
    return _bound(model_dir, requests, plain.round_bf16, 3.0, 5e-3)
