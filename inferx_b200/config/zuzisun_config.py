"""Typed configuration of the Zuzisun design, read from its own ``config.json``.

The file is nested: ``architecture`` (a string), ``vocab``, ``width``, ``embedding.scale``,
``norm.eps`` / ``norm.groups``, and ``layers``, a list with one object per layer: ``type``
(which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (its feed-forward, or null
for a layer without one).  Every size and constant a model of the design can vary is read
from there; a key of the wrong JSON type, an unknown layer type or feed-forward kind, or
sizes that do not fit together are refused with the place named.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError, _Reader

ARCHITECTURE = "Zuzisun"
LATENT = "latent_attention"
DENSE = "dense"


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int            # plain query/key entries per head
    rot_dim: int        # rotated query/key entries per head
    vdim: int
    kv_rank: int
    scale: float
    window: int         # keys a position sees, itself included; 0: all
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[RotaryScaling]


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class ZuzisunLayer:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[DenseMlpConfig]


@dataclass(frozen=True)
class ZuzisunConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    norm_groups: int
    layers: Tuple[ZuzisunLayer, ...]
    torch_dtype: str = "bfloat16"
    architecture: str = ARCHITECTURE
    eos_token_ids: tuple = ()

    ARCHITECTURE = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_json(cls, obj: Mapping[str, Any], where: str = "config.json") -> "ZuzisunConfig":
        r = _Reader(obj, where)
        name = r.string("architecture")
        if name != ARCHITECTURE:
            raise ConfigError(f"{where}: architecture {name!r} is not {ARCHITECTURE!r}")
        emb = _Reader(_object(obj, "embedding", where, {}), f"{where}: embedding")
        norm = _Reader(_object(obj, "norm", where), f"{where}: norm")
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = tuple(_layer(lo, f"{where}: layers[{i}]") for i, lo in enumerate(raw_layers))
        cfg = cls(vocab=r.integer("vocab"), width=r.integer("width"),
                  embedding_scale=emb.number("scale", 1.0), norm_eps=norm.number("eps"),
                  norm_groups=norm.integer("groups", 1), layers=layers,
                  torch_dtype=r.string("torch_dtype", "bfloat16"))
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        def need(ok, msg):
            if not ok:
                raise ConfigError(f"{where}: {msg}")

        need(self.vocab > 0 and self.width > 0, "'vocab' and 'width' must be positive")
        need(self.norm_eps > 0, "'norm.eps' must be positive")
        need(self.norm_groups > 0 and self.width % self.norm_groups == 0,
             f"'width' {self.width} does not split into {self.norm_groups} norm groups")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            at = f"layers[{i}].mixer"
            need(min(m.heads, m.vdim, m.kv_rank) > 0 and m.dim >= 0 and m.rot_dim >= 0
                 and m.dim + m.rot_dim > 0, f"{at}: sizes must be positive")
            need(m.window >= 0, f"{at}: 'mask.size' must not be negative")
            need(m.rot_dims % 2 == 0 and 0 <= m.rot_dims <= m.rot_dim,
                 f"{at}: 'rot.dims' {m.rot_dims} must be even and at most rot_dim {m.rot_dim}")
            need(m.rot_base > 1.0 or m.rot_dims == 0, f"{at}: 'rot.base' must exceed 1")
            if m.rot_scaling is not None:
                sc = m.rot_scaling
                need(sc.factor > 0 and sc.original > 0 and sc.fast > 0 and sc.slow > 0,
                     f"{at}: 'rot.scaling' values must be positive")
            if layer.mlp is not None:
                need(layer.mlp.ff > 0, f"layers[{i}].mlp: 'ff' must be positive")

    def to_json(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale},
               "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "layers": [],
               "torch_dtype": self.torch_dtype}
        for layer in self.layers:
            m = layer.mixer
            rot = {"base": m.rot_base, "dims": m.rot_dims}
            if m.rot_scaling is not None:
                sc = m.rot_scaling
                rot["scaling"] = {"factor": sc.factor, "original": sc.original, "fast": sc.fast,
                                  "slow": sc.slow}
            mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                     "kv_rank": m.kv_rank, "scale": m.scale, "rot": rot}
            if m.window:
                mixer["mask"] = {"size": m.window}
            out["layers"].append({
                "type": layer.type, "mixer": mixer,
                "mlp": None if layer.mlp is None else {"kind": DENSE, "ff": layer.mlp.ff,
                                                       "limit": layer.mlp.limit}})
        return out


def _object(obj, key, where, default=None):
    v = obj.get(key) if isinstance(obj, Mapping) else None
    if v is None:
        if default is None:
            raise ConfigError(f"{where}: required object '{key}' is missing")
        return default
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where}: '{key}' must be an object, got {v!r}")
    return v


def _layer(obj, where) -> ZuzisunLayer:
    if not isinstance(obj, Mapping):
        raise ConfigError(f"{where}: must be an object")
    kind = _Reader(obj, where).string("type")
    if kind != LATENT:
        # an unknown kind of layer is refused, never run as another
        raise ConfigError(f"{where}: unknown layer type {kind!r} (known: {LATENT!r})")
    m = _Reader(_object(obj, "mixer", where), f"{where}.mixer")
    rot_dim = m.integer("rot_dim")
    rot_obj = _object(m.obj, "rot", f"{where}.mixer", {})
    rot = _Reader(rot_obj, f"{where}.mixer.rot")
    scaling = None
    sc_obj = rot_obj.get("scaling") if isinstance(rot_obj, Mapping) else None
    if sc_obj is not None:
        sc = _Reader(_object(rot_obj, "scaling", f"{where}.mixer.rot"), f"{where}.mixer.rot.scaling")
        scaling = RotaryScaling(factor=sc.number("factor"), original=sc.number("original"),
                                fast=sc.number("fast"), slow=sc.number("slow"))
    mask = _Reader(_object(m.obj, "mask", f"{where}.mixer", {}), f"{where}.mixer.mask")
    mixer = LatentMixerConfig(
        heads=m.integer("heads"), dim=m.integer("dim"), rot_dim=rot_dim,
        vdim=m.integer("vdim"), kv_rank=m.integer("kv_rank"), scale=m.number("scale"),
        window=mask.integer("size", 0),
        rot_dims=rot.integer("dims", rot_dim if rot_obj else 0),
        rot_base=rot.number("base", 10000.0), rot_scaling=scaling)
    mlp = None
    if obj.get("mlp") is not None:
        f = _Reader(_object(obj, "mlp", where), f"{where}.mlp")
        fk = f.string("kind")
        if fk != DENSE:
            raise ConfigError(f"{where}.mlp: unknown kind {fk!r} (known: {DENSE!r})")
        mlp = DenseMlpConfig(ff=f.integer("ff"), limit=f.number("limit"))
    return ZuzisunLayer(type=kind, mixer=mixer, mlp=mlp)
