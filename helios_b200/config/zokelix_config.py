"""Typed configuration of the Zokelix design, read from ``config.json``.

The file lists the layers one by one: every entry names its mixer (``latent_attention``
or ``channel_delta``) with the mixer's sizes and its feed-forward (dense, routed, or none),
so two models of the design may differ in every size, in the order of the layers and in
every constant.  Sizes that the file does not give are read off the checkpoint's tensor
shapes (the inner size of the recurrent mixer's two-step projections).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError


def _need(d: Dict[str, Any], key: str, where: str, kind=int):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    v = d[key]
    if kind is int:
        if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
            raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
        return v
    if not isinstance(v, (int, float)) or isinstance(v, bool):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: Optional[YarnScaling]


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int          # unrotated query/key values per head
    rot_dim: int      # rotated query/key values per head (the key part is shared)
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig


@dataclass(frozen=True)
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int] = None    # rows of a1; None until read off the checkpoint
    gate_rank: Optional[int] = None     # rows of g1


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class MoeMlpConfig:
    ff: int
    limit: float
    experts: int
    top: int


@dataclass(frozen=True)
class ZokelixLayer:
    type: str
    mixer: Any
    mlp: Any          # DenseMlpConfig | MoeMlpConfig | None


@dataclass(frozen=True)
class ZokelixConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    layers: Tuple[ZokelixLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_json(cls, cfg: Dict[str, Any]) -> "ZokelixConfig":
        vocab = _need(cfg, "vocab", "the file")
        width = _need(cfg, "width", "the file")
        eps = _need(cfg.get("norm"), "eps", "norm", float)
        layers = cfg.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = layer.get("type") if isinstance(layer, dict) else None
            mx = layer.get("mixer") if isinstance(layer, dict) else None
            if kind == "latent_attention":
                mixer = _latent(mx, where + ".mixer")
            elif kind == "channel_delta":
                mixer = _delta(mx, where + ".mixer")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not supported "
                                  "(latent_attention, channel_delta)")
            out.append(ZokelixLayer(kind, mixer, _mlp(layer.get("mlp"), where + ".mlp")))
        eos = cfg.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(architecture=str(cfg.get("architecture", "Zokelix")), vocab_size=vocab, width=width,
                   norm_eps=eps, layers=tuple(out), eos_token_ids=eos_ids)

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "ZokelixConfig":
        """Fill the sizes the file leaves out from the checkpoint's tensor shapes."""
        layers = []
        for i, layer in enumerate(self.layers):
            mx = layer.mixer
            if isinstance(mx, ChannelDeltaConfig) and (mx.decay_rank is None or mx.gate_rank is None):
                a1, g1 = shapes.get(f"l{i}.mix.a1"), shapes.get(f"l{i}.mix.g1")
                if a1 is None or g1 is None or len(a1) != 2 or len(g1) != 2:
                    raise ConfigError(f"layer {i}: the checkpoint lacks l{i}.mix.a1 / l{i}.mix.g1, whose "
                                      "rows give the inner size of the decay and gate projections")
                mx = replace(mx, decay_rank=mx.decay_rank or int(a1[0]), gate_rank=mx.gate_rank or int(g1[0]))
            layers.append(replace(layer, mixer=mx))
        return replace(self, layers=tuple(layers))


def _latent(mx, where) -> LatentAttentionConfig:
    rot = mx.get("rot") if isinstance(mx, dict) else None
    rot_dim = _need(mx, "rot_dim", where)
    dims = _need(rot, "dims", where + ".rot")
    if dims % 2 or dims > rot_dim:
        raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most rot_dim {rot_dim}")
    sc = rot.get("scaling")
    scaling = None
    if sc:
        scaling = YarnScaling(_need(sc, "factor", where + ".rot.scaling", float),
                              _need(sc, "original", where + ".rot.scaling", float),
                              _need(sc, "fast", where + ".rot.scaling", float),
                              _need(sc, "slow", where + ".rot.scaling", float))
    return LatentAttentionConfig(
        heads=_need(mx, "heads", where), dim=_need(mx, "dim", where), rot_dim=rot_dim,
        vdim=_need(mx, "vdim", where), kv_rank=_need(mx, "kv_rank", where),
        scale=_need(mx, "scale", where, float),
        rot=RotaryConfig(_need(rot, "base", where + ".rot", float), dims, scaling))


def _delta(mx, where) -> ChannelDeltaConfig:
    heads, kv_heads = _need(mx, "heads", where), _need(mx, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.kv_heads {kv_heads} must divide heads {heads}")
    low = mx.get("low_rank")
    return ChannelDeltaConfig(heads=heads, kv_heads=kv_heads, dim=_need(mx, "dim", where),
                              vdim=_need(mx, "vdim", where), conv=_need(mx, "conv", where),
                              decay_rank=low, gate_rank=low)


def _mlp(ml, where):
    if ml is None:
        return None
    kind = ml.get("kind") if isinstance(ml, dict) else None
    if kind == "dense":
        return DenseMlpConfig(_need(ml, "ff", where))
    if kind == "moe":
        ex, ro = ml.get("expert"), ml.get("router")
        experts, top = _need(ro, "experts", where + ".router"), _need(ro, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router.top {top} exceeds experts {experts}")
        return MoeMlpConfig(_need(ex, "ff", where + ".expert"), _need(ex, "limit", where + ".expert", float),
                            experts, top)
    raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported (dense, moe)")
