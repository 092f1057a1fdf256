"""Zuzisun: from the typed config to a ``ModelSpec``.

The only file that knows how this design chooses its parts.  Every layer is the
"sublayer_norm" arrangement (x += norm(mixer(shift(x))); x += norm(ffn(x))) with a
token shift ahead of the mixer, a grouped RMS norm after each sublayer, latent
attention with an interleaved, YaRN-stretched rotation of its rotated part, a sliding
window and a sigmoid output gate, and a clamped GLU feed-forward (or none).  The
residual stream starts as embed[token] * embedding.scale; the head is the embedding
table itself, unscaled.  Tensor names: ``embed``, ``final.norm``, and per layer i
``l<i>.shift``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from ..config.zuzisun_config import ZuzisunConfig
from ..parts.specs import (ClampedGluSpec, GroupedRmsNormSpec, InterleavedRopeSpec,
                           LatentAttentionSpec, LayerSpec, ModelSpec, RunEntry, TokenShiftSpec)

GLU_SIGMOID_SLOPE = 1.702     # fixed by the design, like the 1 added to the linear branch
GLU_UP_SHIFT = 1.0


def build_spec(cfg: ZuzisunConfig) -> ModelSpec:
    norm = GroupedRmsNormSpec(size=cfg.width, eps=cfg.norm_eps, groups=cfg.norm_groups)
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        rope = None
        if m.rot_dims > 0:
            sc = m.rot_scaling
            rope = InterleavedRopeSpec(
                head_dim=m.rot_dim, rotary_dim=m.rot_dims, theta=m.rot_base,
                scaling_factor=sc.factor if sc else 0.0,
                original_context=sc.original if sc else 0.0,
                fast_turns=sc.fast if sc else 32.0, slow_turns=sc.slow if sc else 1.0)
        mixer = LatentAttentionSpec(
            hidden=cfg.width, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim,
            kv_rank=m.kv_rank, scale=m.scale, window=m.window, position=rope,
            latent_eps=cfg.norm_eps, output_gate=True)
        ffn = None
        if layer.mlp is not None:
            ffn = ClampedGluSpec(hidden=cfg.width, intermediate=layer.mlp.ff,
                                 limit=layer.mlp.limit, alpha=GLU_SIGMOID_SLOPE,
                                 up_shift=GLU_UP_SHIFT)
        layers.append(LayerSpec(
            prefix=f"l{i}", input_norm=norm, mixer=mixer, post_norm=norm if ffn else None,
            ffn=ffn, input_norm_name="norm1", mixer_name="mix", post_norm_name="norm2",
            ffn_name="mlp", kind="sublayer_norm", mixer_input=TokenShiftSpec(size=cfg.width),
            mixer_input_name="shift"))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden=cfg.width,
        layers=tuple(layers), schedule=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=norm, tied_head=True, embed_name="embed", final_norm_name="final.norm",
        head_name="embed", embed_scale=cfg.embedding_scale)
