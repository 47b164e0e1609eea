"""Plan of the Zokelix design: a token embedding, post-norm blocks (the norm sits on each
sublayer's output) whose mixer is either attention over a low-rank latent cache or a
gated-delta-rule recurrence, and whose feed-forward is dense (tanh-gelu gate, biases),
routed (sigmoid router, clamped-swish experts) or absent; a final RMS norm and the head.

Every layer's parts are made from that layer's entry of the configuration, so the order of
the layers and all sizes are the file's.  Layers with equal rotary constants share one
encoding (one cos/sin table a step).
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zokelix_config import (ChannelDeltaConfig, DenseMlpConfig, LatentAttentionConfig,
                                     MoeMlpConfig, ZokelixConfig)
from ..parts import ModelPlan, OutputHead, TokenEmbedding, part_class
from ..parts.rotary import yarn_attention_factor, yarn_frequencies


def _encoding(rot, made):
    if rot not in made:
        cls = part_class("position_encoding", "rotary")
        if rot.scaling is None:
            made[rot] = cls(rot.dims, rot.base)
        else:
            s = rot.scaling
            made[rot] = cls(rot.dims, rot.base,
                            inv_freq=yarn_frequencies(rot.dims, rot.base, s.factor, s.original, s.fast, s.slow),
                            attention_factor=yarn_attention_factor(s.factor))
    return made[rot]


def build_zokelix_plan(cfg: ZokelixConfig) -> ModelPlan:
    norm_cls = part_class("norm", "rmsnorm")
    block_cls = part_class("block", "post_norm")
    encodings = {}
    layers, prefixes = [], []
    for i, layer in enumerate(cfg.layers):
        mx = layer.mixer
        if isinstance(mx, LatentAttentionConfig):
            mixer = part_class("mixer", "latent_attention")(
                cfg.width, mx.heads, mx.dim, mx.rot_dim, mx.vdim, mx.kv_rank, mx.scale, cfg.norm_eps,
                _encoding(mx.rot, encodings))
        elif isinstance(mx, ChannelDeltaConfig):
            if mx.decay_rank is None or mx.gate_rank is None:
                raise ValueError(f"layer {i}: the inner sizes of the decay and gate projections are "
                                 "neither in config.json ('low_rank') nor read off a checkpoint")
            mixer = part_class("mixer", "gated_delta")(
                cfg.width, mx.heads, mx.kv_heads, mx.dim, mx.vdim, mx.conv, mx.decay_rank, mx.gate_rank,
                cfg.norm_eps)
        else:
            raise ValueError(f"layer {i}: unknown mixer configuration {type(mx).__name__}")
        ml = layer.mlp
        if ml is None:
            ffn = ffn_norm = None
        else:
            if isinstance(ml, DenseMlpConfig):
                ffn = part_class("feed_forward", "gated_mlp")(
                    cfg.width, ml.ff, activation="gelu_tanh", bias=True, names=("gate", "up", "down"))
            elif isinstance(ml, MoeMlpConfig):
                ffn = part_class("feed_forward", "routed_experts")(
                    cfg.width, ml.ff, ml.experts, ml.top, ml.limit)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward configuration {type(ml).__name__}")
            ffn_norm = norm_cls(cfg.width, cfg.norm_eps, tensor_name="")
        layers.append(block_cls(mixer, norm_cls(cfg.width, cfg.norm_eps, tensor_name=""), ffn, ffn_norm))
        prefixes.append(f"l{i}.")
    return ModelPlan(
        config=cfg,
        embedding=TokenEmbedding(cfg.vocab_size, cfg.width, tensor_name=""),
        position=None,
        layers=layers,
        layer_prefixes=prefixes,
        final_norm=norm_cls(cfg.width, cfg.norm_eps, tensor_name=""),
        head=OutputHead(cfg.vocab_size, cfg.width, tensor_name=""),
        embedding_prefix="embed",
        final_norm_prefix="final.norm",
        head_prefix="head",
        benign_suffixes=(),
    )


def _toy_config(sizes):
    """config.json of a small model of the design from the sizes ``make-toy-model`` takes:
    the layers alternate the two mixers; the first feed-forward is dense, the others routed."""
    width = sizes["hidden_size"]
    heads = sizes["heads"]
    hd = sizes.get("head_dim") or max(8, (width // heads) // 2 * 2)
    inner = sizes.get("intermediate_size") or 2 * width
    rot = {"base": sizes["rope_theta"], "dims": hd}
    if sizes.get("rope_scaling"):
        f, lo, hi, orig = sizes["rope_scaling"]
        rot["scaling"] = {"factor": f, "fast": hi, "slow": lo, "original": int(orig)}
    layers = []
    for i in range(sizes["layers"]):
        if i % 2 == 0:
            mixer = {"heads": heads, "dim": hd, "rot_dim": hd, "vdim": hd, "kv_rank": 2 * hd,
                     "scale": (2 * hd) ** -0.5, "rot": rot}
            kind = "latent_attention"
        else:
            mixer = {"heads": heads, "kv_heads": sizes["kv_heads"], "dim": hd, "vdim": hd, "conv": 4,
                     "low_rank": 8}
            kind = "channel_delta"
        mlp = {"kind": "dense", "ff": inner} if i == 0 else \
            {"kind": "moe", "expert": {"ff": max(8, inner // 4), "limit": 7.0},
             "router": {"experts": 4, "top": 2}}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Zokelix", "vocab": sizes["vocab_size"], "width": width,
            "norm": {"eps": sizes["rms_eps"]}, "layers": layers}


register_architecture("Zokelix", ZokelixConfig.from_json, build_zokelix_plan, toy_config=_toy_config,
                      sizes_from_tensors=lambda cfg, shapes: cfg.with_tensor_shapes(shapes), replace=True)
