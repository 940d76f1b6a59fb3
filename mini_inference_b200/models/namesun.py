"""Namesun: configuration -> ModelSpec.

A decoder whose layers are chosen one by one from two mixers (softmax attention inside blocks of
positions, with a sink term and unit-norm queries and keys; a retention recurrence with a fixed decay
per head), each followed by a dense or routed feed-forward (or none).  A sublayer reads the
residual stream itself; its OUTPUT is normed, multiplied by a layer-scale vector and one number,
and added to the stream, which is kept in float32.  Attention layers that say so blend the
values of the first such layer into their own.
Tensor names are the checkpoint's own: embed, l<i>.norm1, l<i>.ls1, l<i>.mix.*, l<i>.norm2, l<i>.ls2,
l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

from ..config.namesun_config import NamesunConfig
from ..config.registry import register_architecture
from ..config.spec import ExecStep, LayerSpec, ModelSpec, PartSpec


def build_spec(cfg: NamesunConfig) -> ModelSpec:
    none = PartSpec.of("none")
    out_norm = PartSpec.of("out_rmsnorm", size=cfg.width, eps=cfg.norm_eps, mult=cfg.residual_mult, layer_scale=True)
    layers, value_source = [], None
    for i, layer in enumerate(cfg.layers):
        m, p = layer.mixer_dict(), f"l{i}."
        names = {"norm1.weight": p + "norm1", "norm1.scale": p + "ls1"}
        position = none
        if layer.type == "attention":
            role = None
            if m.get("v_mix"):                           # the first such layer lends its values, the others blend them in
                role = "source" if value_source is None else "blend"
                value_source = i if value_source is None else value_source
            mask = m.get("mask") or {}
            mixer = PartSpec.of("sink_attention", hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
                                key_dim=m["dim"], value_dim=m["vdim"], scale=m["scale"], unit_norm_eps=cfg.norm_eps,
                                block_size=mask.get("size"), sink=True, value_mix=role)
            tensors = ("q", "k", "v", "o") + (("vmix",) if role else ())
        else:
            mixer = PartSpec.of("retention", hidden_size=cfg.width, num_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
                                decay=tuple(m["decay"]), out_norm_eps=cfg.norm_eps)
            if m["rot"]["dims"] > 0:
                position = PartSpec.of("rotary_half", dims=m["rot"]["dims"], theta=m["rot"]["base"])
            tensors = ("q", "k", "v", "g", "o")
        names.update({f"mixer.{t}": p + "mix." + t for t in tensors})
        parts = dict(mixer=mixer, norm1=out_norm, position=position)
        block = "outnorm_mixer"
        if layer.mlp is not None:
            block = "outnorm"
            names.update({"norm2.weight": p + "norm2", "norm2.scale": p + "ls2"})
            if layer.mlp.kind == "dense":
                ff = PartSpec.of("swiglu", hidden_size=cfg.width, intermediate_size=layer.mlp.ff)
                names.update({"feed_forward.gate_proj": p + "mlp.gate", "feed_forward.up_proj": p + "mlp.up",
                              "feed_forward.down_proj": p + "mlp.down"})
            else:
                mlp = layer.mlp
                ff = PartSpec.of("routed_experts", hidden_size=cfg.width, num_experts=mlp.experts, top=mlp.top,
                                 groups=mlp.groups, expert_size=mlp.ff, limit=mlp.limit, gate_slope=1.702,
                                 shared_size=mlp.shared[0] if mlp.shared else None,
                                 shared_limit=mlp.shared[1] if mlp.shared else None)
                names.update({"feed_forward.router": p + "mlp.router", "feed_forward.correction": p + "mlp.correction"})
                for e in range(mlp.experts):
                    names.update({f"feed_forward.e{e}.{t}": f"{p}mlp.e{e}.{t}" for t in ("gate", "up", "down")})
                if mlp.shared:
                    names.update({f"feed_forward.shared.{t}": f"{p}mlp.shared.{t}" for t in ("gate", "up", "down")})
            parts.update(norm2=out_norm, feed_forward=ff)
        layers.append(LayerSpec.of(block, names, **parts))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers), order=tuple(ExecStep(i) for i in range(len(layers))),
        final_norm=PartSpec.of("stream_rmsnorm", size=cfg.width, eps=cfg.norm_eps), embedding_name="embed",
        final_norm_name="final.norm", lm_head_name="head", max_position=cfg.max_position, residual="float32")


register_architecture("Namesun", "Namesun (block-local sink attention / retention layers, routed experts, output norms, float32 stream)",
                      NamesunConfig, build_spec)
