"""Naditar: configuration -> ModelSpec.

A decoder whose layers are chosen one by one from three mixers (a decayed linear-attention
recurrence, a gated delta-rule recurrence with short convolutions, and latent attention with a
compressed cache), each followed by an optional dense feed-forward with a polynomial norm
activation; every norm of the stream is a root-mean-square norm with ONE learned number; the
residual stream is kept in float32; a span of layers may run several times with the same
weights, each repetition with a cache or state of its own and a learned vector added before it.
Tensor names are the checkpoint's own: embed, embed.norm, loop.step, l<i>.norm1, l<i>.mix.*,
l<i>.norm2, l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

from ..config.naditar_config import NaditarConfig
from ..config.registry import register_architecture
from ..config.spec import ExecStep, LayerSpec, ModelSpec, PartSpec

_MIXER_TENSORS = {
    "lightning": ("q", "k", "v", "g", "o", "norm"),
    "channel_delta": ("q", "q.conv", "k", "k.conv", "v", "v.conv", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o"),
    "latent_attention": ("q", "dkv", "dkv.norm", "uk", "uv", "g", "o"),
}


def execution_order(num_layers: int, loop):
    """Layers before the repeated span once, the span `times` times (the first layer of each repetition adds that
    repetition's vector), the rest once."""
    if loop is None:
        return tuple(ExecStep(i) for i in range(num_layers))
    start, stop, times = loop
    order = [ExecStep(i) for i in range(start)]
    for t in range(times):
        order += [ExecStep(i, add_row=t if i == start else None) for i in range(start, stop)]
    return tuple(order + [ExecStep(i) for i in range(stop, num_layers)])


def build_spec(cfg: NaditarConfig) -> ModelSpec:
    norm = PartSpec.of("scalar_rmsnorm", eps=cfg.norm_eps)
    none = PartSpec.of("none")
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer_dict()
        position = none
        if layer.type == "lightning":
            mixer = PartSpec.of("lightning", hidden_size=cfg.width, num_heads=m["heads"], key_dim=m["dim"],
                                value_dim=m["vdim"], decay=tuple(m["decay"]), out_norm_eps=cfg.norm_eps)
        elif layer.type == "channel_delta":
            mixer = PartSpec.of("channel_delta", hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
                                key_dim=m["dim"], value_dim=m["vdim"], conv_taps=m["conv"], out_norm_eps=cfg.norm_eps,
                                unit_eps=1e-6, decay_rank=m.get("decay_rank", -1), gate_rank=m.get("gate_rank", -1))
        else:
            mixer = PartSpec.of("latent_attention", hidden_size=cfg.width, num_heads=m["heads"], nope_dim=m["dim"],
                                rot_dim=m["rot_dim"], value_dim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"],
                                latent_norm_eps=cfg.norm_eps)
            position = PartSpec.of("rotary_interleaved", dims=m["rot"]["dims"], theta=m["rot"]["base"])
        p = f"l{i}."
        names = {"norm1.weight": p + "norm1"}
        names.update({f"mixer.{t}": p + "mix." + t for t in _MIXER_TENSORS[layer.type]})
        parts = dict(mixer=mixer, norm1=norm, position=position)
        block = "prenorm_mixer"
        if layer.ff is not None:
            block = "prenorm"
            parts.update(norm2=norm, feed_forward=PartSpec.of("polynorm_mlp", hidden_size=cfg.width,
                                                              intermediate_size=layer.ff, eps=cfg.norm_eps))
            names.update({"norm2.weight": p + "norm2", "feed_forward.up": p + "mlp.up",
                          "feed_forward.down": p + "mlp.down", "feed_forward.act": p + "mlp.act"})
        layers.append(LayerSpec.of(block, names, **parts))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers),
        order=execution_order(len(layers), cfg.loop), final_norm=norm, embedding_name="embed",
        final_norm_name="final.norm", lm_head_name="head", max_position=cfg.max_position,
        embedding_norm=norm, embedding_norm_name="embed.norm",
        pass_vectors_name="loop.step" if cfg.loop is not None else None,
        pass_vectors_rows=cfg.loop[2] if cfg.loop is not None else 0, residual="float32")


register_architecture("Naditar", "Naditar (lightning / channel delta / latent attention layers, looped span, float32 stream)",
                      NaditarConfig, build_spec)
