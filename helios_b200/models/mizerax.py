"""Plan of the Mizerax design: token embedding plus a learned vector per position; parallel
blocks (one layer norm, whose output both the mixer and the feed-forward read; per-channel
factors on both outputs and one multiplier on their sum); the mixer is grouped-query attention
with normed queries and keys, a query temperature by position, a linear distance bias, a sink
in the softmax and a gate per head; the feed-forward is routed (softmax router with a
correction for the choice, experts without tensors that return their input, an expert every
token runs) or absent; a stretch of the layers may run several times over with the same
weights, each pass with a cache of its own and the embedded input mixed into the stream
before its first layer; a final layer norm and the embedding table as the head.

Every layer's parts are made from that layer's entry of the configuration, so the order of
the layers and all sizes are the file's.
"""
from __future__ import annotations

from ..config.mizerax_config import MizeraxConfig, fill_from_tensor_shapes
from ..config.registry import register_architecture
from ..parts import ModelPlan, OutputHead, Run, TokenEmbedding, distance_slopes, part_class
from ..parts.stream import StreamInputMix

#: exponent of the distance bias: head h of H has the slope 2 ^ (-8 (h + 1) / H)
SLOPE_EXPONENT = 8.0
LOOP_STAGE = "loop."


def build_mizerax_plan(cfg: MizeraxConfig) -> ModelPlan:
    if cfg.max_positions is None:
        raise ValueError("the number of learned positions is neither in config.json ('max_positions') "
                         "nor read off a checkpoint")
    norm_cls = part_class("norm", "layernorm")
    block_cls = part_class("block", "parallel")
    mixer_cls = part_class("mixer", "sink_gqa_attention")
    ffn_cls = part_class("feed_forward", "routed_experts")

    def norm():
        return norm_cls(cfg.width, cfg.norm_eps, weight_name="", bias_name=".b")

    layers, prefixes = [], []
    for i, layer in enumerate(cfg.layers):
        mx = layer.mixer
        mixer = mixer_cls(cfg.width, mx.heads, mx.kv_heads, mx.dim, mx.scale, value_dim=mx.vdim,
                          qk_norm=True, eps=cfg.norm_eps,
                          q_temperature=(mx.q_temp.coef, mx.q_temp.every) if mx.q_temp else None,
                          slopes=distance_slopes(mx.heads, SLOPE_EXPONENT), sink=True, head_gate=True)
        ml = layer.mlp
        ffn = None
        if ml is not None:
            ffn = ffn_cls(cfg.width, ml.ff, ml.experts, ml.top, router="softmax", correction=True,
                          weight_on="output", activation="silu", identity=ml.identity,
                          shared_inner=ml.shared_ff)
        layers.append(block_cls(norm(), mixer, ffn, mult=cfg.residual_mult, layer_scale=True))
        prefixes.append(f"l{i}.")
    schedule = [Run(i, before=LOOP_STAGE if begins else None) for i, begins in cfg.layer_runs()]
    looped = any(begins for _i, begins in cfg.layer_runs())
    return ModelPlan(
        config=cfg,
        embedding=TokenEmbedding(cfg.vocab_size, cfg.width, tensor_name=""),
        position=part_class("position_encoding", "learned")(cfg.max_positions, cfg.width, tensor_name=""),
        layers=layers,
        layer_prefixes=prefixes,
        final_norm=norm(),
        head=OutputHead(cfg.vocab_size, cfg.width, tensor_name=""),
        schedule=schedule,
        embedding_prefix="embed",
        position_prefix="pos",
        final_norm_prefix="final.norm",
        head_prefix="head",
        tied={"head": "embed"},
        # a file whose loop runs nothing may still bring the loop's matrix
        benign_suffixes=() if looped else (LOOP_STAGE + "in",),
        stages={LOOP_STAGE: StreamInputMix(cfg.width, tensor_name="in")} if looped else {},
    )


def _toy_config(sizes):
    """config.json of a small model of the design from the sizes ``make-toy-model`` takes: the
    middle layers run twice; every layer but the last has a routed feed-forward."""
    width = sizes["hidden_size"]
    heads = sizes["heads"]
    hd = sizes.get("head_dim") or max(8, (width // heads) // 2 * 2)
    inner = sizes.get("intermediate_size") or 2 * width
    n = sizes["layers"]
    layers = []
    for i in range(n):
        mixer = {"heads": heads, "kv_heads": sizes["kv_heads"], "dim": hd, "vdim": hd,
                 "scale": hd ** -0.5, "q_temp": {"coef": 0.25, "every": 64}}
        mlp = None if (i == n - 1 and n > 1) else \
            {"kind": "moe", "expert": {"ff": max(8, inner // 4)},
             "router": {"experts": 4, "identity": 1, "top": 2}, "shared": {"ff": max(8, inner // 2)}}
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Mizerax", "vocab": sizes["vocab_size"], "width": width,
           "max_positions": sizes["max_pos"], "norm": {"eps": sizes["rms_eps"]}, "residual_mult": 0.8,
           "layers": layers}
    if n >= 3:
        cfg["loop"] = {"start": 1, "stop": n - 1, "times": 2}
    return cfg


register_architecture("Mizerax", MizeraxConfig.from_json, build_mizerax_plan, toy_config=_toy_config,
                      sizes_from_tensors=fill_from_tensor_shapes, replace=True)
