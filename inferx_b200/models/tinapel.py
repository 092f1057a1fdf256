"""Tinapel: from the typed config to a ``ModelSpec``.

The only file that knows how this design chooses its parts.  Every layer is the
"parallel" arrangement, x += mixer(norm1(x)) + ffn(norm2(x)), with RMS norms whose
weights are stored around zero.  A layer's mixer is wkv time mixing, gated linear
attention or softmax attention whose values are its keys; its feed-forward a mixture of
experts with renormalised, scaled weights and an ungated shared expert, or none.  The
stream starts as embed[token] * embedding.scale plus a sinusoidal position vector; the
head is the embedding table itself, unscaled.  Layers loop.start .. loop.stop-1 run
loop.times times in a row with the same weights, every pass with caches and state of its
own; ahead of every pass row t of ``loop.step`` is added to the stream, and ahead of every
pass but the first the embedding output as well.  Tensor names: ``embed``,
``final.norm``, ``loop.step``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from ..config.tinapel_config import ATTENTION, GLA, WKV, TinapelConfig
from ..parts.specs import (GatedLinearAttentionSpec, LayerSpec, ModelSpec, MoeSpec, RmsNormSpec,
                           RunEntry, SinusoidSpec, StreamAddSpec, SwiGluSpec,
                           TiedKvAttentionSpec, WkvSpec)

SINUSOID_BASE = 10000.0       # fixed by the design
LOOP_TABLE = "loop.step"
_EXPERT = ("gate", "up", "down")


def _mixer(cfg: TinapelConfig, layer):
    m = layer.mixer
    if layer.type == WKV:
        return WkvSpec(hidden=cfg.width, heads=m.heads, dim=m.dim, norm_eps=cfg.norm_eps,
                       decay_rank=m.rank)
    if layer.type == GLA:
        return GatedLinearAttentionSpec(
            hidden=cfg.width, heads=m.heads, dim=m.dim, vdim=m.vdim, tau=m.tau,
            q_scale=float(m.dim) ** -0.5, norm_eps=cfg.norm_eps, decay_rank=m.rank)
    assert layer.type == ATTENTION
    return TiedKvAttentionSpec(
        hidden=cfg.width, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
        norm_eps=cfg.norm_eps, softcap=m.softcap, temp_coef=m.temp_coef,
        temp_every=m.temp_every, window=0)


def _ffn(cfg: TinapelConfig, f):
    if f is None:
        return None
    shared = (SwiGluSpec(hidden=cfg.width, intermediate=f.shared_ff, names=_EXPERT)
              if f.shared_ff else None)
    return MoeSpec(hidden=cfg.width, num_experts=f.experts, top_k=f.top,
                   expert_intermediate=f.expert_ff, renormalize=True, routed_scale=f.scale,
                   shared=shared, shared_gated=False, shared_name="shared",
                   router_name="router",
                   expert_names=tuple("e{e}." + n for n in _EXPERT))


def build_spec(cfg: TinapelConfig) -> ModelSpec:
    norm = RmsNormSpec(size=cfg.width, eps=cfg.norm_eps, gain_offset=1.0, suffix="")
    layers = []
    for i, layer in enumerate(cfg.layers):
        ffn = _ffn(cfg, layer.mlp)
        layers.append(LayerSpec(
            prefix=f"l{i}", input_norm=norm, mixer=_mixer(cfg, layer),
            post_norm=norm if ffn is not None else None, ffn=ffn, input_norm_name="norm1",
            mixer_name="mix", post_norm_name="norm2", ffn_name="mlp", kind="parallel"))
    n, a, b = len(layers), cfg.loop_start, cfg.loop_stop
    if not cfg.has_loop:
        schedule = [RunEntry(i) for i in range(n)]
    else:
        schedule = [RunEntry(i) for i in range(a)]
        for t in range(cfg.loop_times):
            for i in range(a, b):
                before = (StreamAddSpec(table=LOOP_TABLE, rows=cfg.loop_times, row=t,
                                        embedding=t > 0) if i == a else None)
                schedule.append(RunEntry(i, cache_copy=t, before=before))
        schedule += [RunEntry(i) for i in range(b, n)]
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden=cfg.width,
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, tied_head=True,
        embed_name="embed", final_norm_name="final.norm", head_name="embed",
        embed_scale=cfg.embedding_scale,
        embed_position=SinusoidSpec(size=cfg.width, base=SINUSOID_BASE))
