"""Typed configuration of the Tinapel design, read from its own ``config.json``.

Top level: ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``layers`` (one object per layer: ``type`` names the mixer - "wkv", "gla" or "attention" -,
``mixer`` holds its sizes and constants, ``mlp`` its feed-forward or null) and ``loop``
(``start``, ``stop``, ``times``: layers start..stop-1 run ``times`` times in a row).  Every
size and constant a model of the design can vary is read from there; what has a natural
"off" may be absent (no loop, no query temperature, no squashing of scores, no shared
expert).  The inner size of a decay's low-rank product is not a key of the design: the
checkpoint's tensors give it; ``mixer.rank`` is read only so that a folder of random
weights can be written from a configuration alone.  A key of the wrong JSON type, an
unknown layer type or feed-forward kind, or sizes that do not fit are refused with the
place named.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError, _Reader

ARCHITECTURE = "Tinapel"
WKV, GLA, ATTENTION = "wkv", "gla", "attention"
MOE = "moe"


@dataclass(frozen=True)
class TinapelMixer:
    heads: int
    dim: int                  # key (and query) entries per head
    vdim: int                 # value entries per head
    rank: int = 0             # inner size of the decay's low-rank product; 0: the checkpoint's
    tau: float = 1.0          # gla: the decay is sigmoid(z)^(1/tau)
    kv_heads: int = 0         # attention
    scale: float = 1.0        # attention: factor on q . k
    softcap: float = 0.0      # attention: scores become softcap * tanh(score / softcap); 0: not
    temp_coef: float = 0.0    # attention: query temperature 1 + coef * ln(floor((p+1)/every) + 1)
    temp_every: int = 0


@dataclass(frozen=True)
class TinapelMlp:
    experts: int
    top: int
    scale: float
    expert_ff: int
    shared_ff: int            # 0: no shared expert


@dataclass(frozen=True)
class TinapelLayer:
    type: str
    mixer: TinapelMixer
    mlp: Optional[TinapelMlp]


@dataclass(frozen=True)
class TinapelConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[TinapelLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1       # 1 with start == stop: no loop
    torch_dtype: str = "bfloat16"
    architecture: str = ARCHITECTURE
    eos_token_ids: tuple = ()

    ARCHITECTURE = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start

    @classmethod
    def from_json(cls, obj: Mapping[str, Any], where: str = "config.json") -> "TinapelConfig":
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
        start = stop = 0
        times = 1
        if obj.get("loop") is not None:
            lp = _Reader(_object(obj, "loop", where), f"{where}: loop")
            start, stop, times = lp.integer("start"), lp.integer("stop"), lp.integer("times")
        cfg = cls(vocab=r.integer("vocab"), width=r.integer("width"),
                  embedding_scale=emb.number("scale", 1.0), norm_eps=norm.number("eps"),
                  layers=layers, loop_start=start, loop_stop=stop, loop_times=times,
                  torch_dtype=r.string("torch_dtype", "bfloat16"))
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        def need(ok, msg):
            if not ok:
                raise ConfigError(f"{where}: {msg}")

        need(self.vocab > 0 and self.width > 0, "'vocab' and 'width' must be positive")
        need(self.norm_eps > 0, "'norm.eps' must be positive")
        need(0 <= self.loop_start <= self.loop_stop <= len(self.layers) and self.loop_times >= 1,
             f"'loop' {self.loop_start}..{self.loop_stop} x {self.loop_times} does not fit "
             f"{len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            m, at = layer.mixer, f"layers[{i}].mixer"
            need(min(m.heads, m.dim, m.vdim) > 0 and m.rank >= 0, f"{at}: sizes must be positive")
            if layer.type == GLA:
                need(m.tau > 0, f"{at}: 'tau' must be positive")
            if layer.type == ATTENTION:
                need(m.kv_heads > 0 and m.heads % m.kv_heads == 0,
                     f"{at}: {m.heads} heads do not split over {m.kv_heads} key/value heads")
                need(m.vdim == m.dim, f"{at}: the values are the keys, so 'vdim' {m.vdim} "
                                      f"must equal 'dim' {m.dim}")
                need(m.softcap >= 0 and m.temp_every >= 0, f"{at}: 'softcap' and 'q_temp.every' "
                                                           "must not be negative")
            if layer.mlp is not None:
                f = layer.mlp
                need(f.experts > 0 and 0 < f.top <= f.experts and f.expert_ff > 0
                     and f.shared_ff >= 0,
                     f"layers[{i}].mlp: {f.top} of {f.experts} experts of width {f.expert_ff}")

    def to_json(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "layers": [], "torch_dtype": self.torch_dtype}
        if self.has_loop:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop,
                           "times": self.loop_times}
        for layer in self.layers:
            m = layer.mixer
            mixer = {"heads": m.heads, "dim": m.dim}
            if m.rank and layer.type != ATTENTION:
                mixer["rank"] = m.rank
            if layer.type == GLA:
                mixer.update(vdim=m.vdim, tau=m.tau)
            if layer.type == ATTENTION:
                mixer.update(vdim=m.vdim, kv_heads=m.kv_heads, scale=m.scale)
                if m.softcap:
                    mixer["softcap"] = m.softcap
                if m.temp_every:
                    mixer["q_temp"] = {"coef": m.temp_coef, "every": m.temp_every}
            mlp = None
            if layer.mlp is not None:
                f = layer.mlp
                mlp = {"kind": MOE, "expert": {"ff": f.expert_ff},
                       "router": {"experts": f.experts, "top": f.top, "scale": f.scale}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            out["layers"].append({"type": layer.type, "mixer": mixer, "mlp": mlp})
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


def _layer(obj, where) -> TinapelLayer:
    if not isinstance(obj, Mapping):
        raise ConfigError(f"{where}: must be an object")
    kind = _Reader(obj, where).string("type")
    if kind not in (WKV, GLA, ATTENTION):
        # an unknown kind of layer is refused, never run as another
        raise ConfigError(f"{where}: unknown layer type {kind!r} "
                          f"(known: {WKV!r}, {GLA!r}, {ATTENTION!r})")
    m = _Reader(_object(obj, "mixer", where), f"{where}.mixer")
    heads, dim = m.integer("heads"), m.integer("dim")
    if kind == WKV:
        mixer = TinapelMixer(heads=heads, dim=dim, vdim=dim, rank=m.integer("rank", 0))
    elif kind == GLA:
        mixer = TinapelMixer(heads=heads, dim=dim, vdim=m.integer("vdim", dim),
                             rank=m.integer("rank", 0), tau=m.number("tau"))
    else:
        coef, every = 0.0, 0
        if m.obj.get("q_temp") is not None:
            qt = _Reader(_object(m.obj, "q_temp", f"{where}.mixer"), f"{where}.mixer.q_temp")
            coef, every = qt.number("coef"), qt.integer("every")
        mixer = TinapelMixer(heads=heads, dim=dim, vdim=m.integer("vdim", dim),
                             kv_heads=m.integer("kv_heads", heads), scale=m.number("scale"),
                             softcap=m.number("softcap", 0.0), temp_coef=coef, temp_every=every)
    mlp = None
    if obj.get("mlp") is not None:
        f = _Reader(_object(obj, "mlp", where), f"{where}.mlp")
        fk = f.string("kind")
        if fk != MOE:
            raise ConfigError(f"{where}.mlp: unknown kind {fk!r} (known: {MOE!r})")
        ex = _Reader(_object(f.obj, "expert", f"{where}.mlp"), f"{where}.mlp.expert")
        ro = _Reader(_object(f.obj, "router", f"{where}.mlp"), f"{where}.mlp.router")
        shared_ff = 0
        if f.obj.get("shared") is not None:
            shared_ff = _Reader(_object(f.obj, "shared", f"{where}.mlp"),
                                f"{where}.mlp.shared").integer("ff")
        mlp = TinapelMlp(experts=ro.integer("experts"), top=ro.integer("top"),
                         scale=ro.number("scale", 1.0), expert_ff=ex.integer("ff"),
                         shared_ff=shared_ff)
    return TinapelLayer(type=kind, mixer=mixer, mlp=mlp)
