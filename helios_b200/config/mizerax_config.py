"""Typed configuration of the Mizerax design, read from ``config.json``.

The file lists the layers one by one (mixer sizes, feed-forward or none), gives the
stretch of layers that is run several times over with the same weights (``loop``), the
multiplier on every layer's output (``residual_mult``), the number of learned positions
and the norm's eps.  Two models of the design may differ in every size, in the order of
the layers and in every constant; nothing here has a default that stands for a value of
some particular model.  Optional pieces (query temperature, identity experts, shared
expert, the loop itself, a layer's feed-forward) are absent when the file leaves them out
or gives null.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError
from .zokelix_config import _need


@dataclass(frozen=True)
class QueryTemperature:
    coef: float
    every: int


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: Optional[QueryTemperature]


@dataclass(frozen=True)
class RoutedMlpConfig:
    ff: int                 # inner size of a routed expert
    experts: int            # experts with tensors
    identity: int           # router outputs beyond them whose expert returns its input
    top: int
    shared_ff: Optional[int]    # inner size of the expert every token runs; None: no such expert


@dataclass(frozen=True)
class MizeraxLayer:
    type: str
    mixer: SinkAttentionConfig
    mlp: Optional[RoutedMlpConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class MizeraxConfig:
    architecture: str
    vocab_size: int
    width: int
    max_positions: Optional[int]      # None until read off the checkpoint (rows of the position table)
    norm_eps: float
    residual_mult: float
    layers: Tuple[MizeraxLayer, ...]
    loop: Optional[LoopConfig]
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    def layer_runs(self):
        """(layer, begins a pass of the loop) in the order the layers run: the layers before
        the loop once, the loop's layers ``times`` times over, the rest once."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        a, b, times = self.loop.start, self.loop.stop, self.loop.times
        runs = [(i, False) for i in range(a)]
        for _ in range(times):
            runs += [(i, i == a) for i in range(a, b)]
        return runs + [(i, False) for i in range(b, n)]

    @classmethod
    def from_json(cls, cfg: Dict[str, Any]) -> "MizeraxConfig":
        vocab = _need(cfg, "vocab", "the file")
        width = _need(cfg, "width", "the file")
        # the number of learned positions may be left to the position table's shape
        max_pos = _need(cfg, "max_positions", "the file") if cfg.get("max_positions") is not None else None
        eps = _need(cfg.get("norm"), "eps", "norm", float)
        mult = _need(cfg, "residual_mult", "the file", float) if "residual_mult" in cfg else 1.0
        layers = cfg.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind != "attention":
                raise ConfigError(f"config.json: {where}.type {kind!r} is not supported (attention)")
            out.append(MizeraxLayer(kind, _attention(layer.get("mixer"), where + ".mixer"),
                                    _mlp(layer.get("mlp"), where + ".mlp")))
        loop = _loop(cfg.get("loop"), len(out))
        eos = cfg.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(architecture=str(cfg.get("architecture", "Mizerax")), vocab_size=vocab, width=width,
                   max_positions=max_pos, norm_eps=eps, residual_mult=mult, layers=tuple(out), loop=loop,
                   eos_token_ids=eos_ids)


def fill_from_tensor_shapes(cfg: MizeraxConfig, shapes: Dict[str, Tuple[int, ...]]) -> MizeraxConfig:
    """Sizes the file leaves out, read off the checkpoint's tensor shapes."""
    if cfg.max_positions is None:
        pos = shapes.get("pos")
        if pos is None or len(pos) != 2:
            raise ConfigError("config.json has no 'max_positions' and the checkpoint no position table 'pos'")
        cfg = replace(cfg, max_positions=int(pos[0]))
    return cfg


def _attention(mx, where) -> SinkAttentionConfig:
    heads, kv_heads = _need(mx, "heads", where), _need(mx, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.kv_heads {kv_heads} must divide heads {heads}")
    qt = mx.get("q_temp")
    temp = None
    if qt:
        temp = QueryTemperature(_need(qt, "coef", where + ".q_temp", float), _need(qt, "every", where + ".q_temp"))
    return SinkAttentionConfig(heads=heads, kv_heads=kv_heads, dim=_need(mx, "dim", where),
                               vdim=_need(mx, "vdim", where), scale=_need(mx, "scale", where, float),
                               q_temp=temp)


def _mlp(ml, where) -> Optional[RoutedMlpConfig]:
    if ml is None:
        return None
    kind = ml.get("kind") if isinstance(ml, dict) else None
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported (moe)")
    ro = ml.get("router")
    experts, top = _need(ro, "experts", where + ".router"), _need(ro, "top", where + ".router")
    identity = ro.get("identity") or 0
    if not isinstance(identity, int) or isinstance(identity, bool) or identity < 0:
        raise ConfigError(f"config.json: {where}.router.identity must be a count, got {identity!r}")
    if top > experts + identity:
        raise ConfigError(f"config.json: {where}.router.top {top} exceeds the {experts + identity} router outputs")
    shared = ml.get("shared")
    return RoutedMlpConfig(ff=_need(ml.get("expert"), "ff", where + ".expert"), experts=experts,
                           identity=identity, top=top,
                           shared_ff=_need(shared, "ff", where + ".shared") if shared else None)


def _loop(lp, n_layers: int) -> Optional[LoopConfig]:
    if not lp:
        return None
    for key in ("start", "stop", "times"):
        v = lp.get(key) if isinstance(lp, dict) else None
        if not isinstance(v, int) or isinstance(v, bool) or v < 0:
            raise ConfigError(f"config.json: loop.{key} must be a count, got {v!r}")
    start, stop, times = lp["start"], lp["stop"], lp["times"]
    if not start <= stop <= n_layers:
        raise ConfigError(f"config.json: loop {start}..{stop} x {times} does not fit {n_layers} layers")
    # an empty stretch runs nothing, whatever the count; a count of 0 leaves the stretch's layers out
    return LoopConfig(start, stop, times) if stop > start else None
