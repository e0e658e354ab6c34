"""Typed configuration of the Zisesun decoder, read from config.json keys.

A Zisesun model is a list of layers, each with one of two token mixers and an optional routed
feed-forward, around one residual stream or several (hyper-connections).  config.json carries:

* ``architecture`` "Zisesun", ``vocab``, ``width``, ``max_positions``, ``norm.eps``;
* ``streams`` (absent: one plain residual stream);
* ``layers``: per layer ``type`` ("attention" or "lightning"), ``mixer`` (its sizes and constants),
  ``mlp`` (null, or ``kind`` "moe" with ``expert.ff``, ``router.experts``, ``router.top``) and
  optionally ``weights_of``: the index of the layer whose tensors this layer runs with (its cache
  and state are its own).

Every size and constant comes from here; this module is the only place that knows the key names.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .model_config import ConfigError


def _get(raw: dict[str, Any], key: str, kind: type | tuple[type, ...], where: str) -> Any:
    if not isinstance(raw, dict) or key not in raw:
        raise ConfigError(f"config.json: {where}: required key {key!r} is missing")
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config.json: {where}: key {key!r} must be {kind}, got {value!r}")
    return value


def _count(raw: dict[str, Any], key: str, where: str) -> int:
    value = _get(raw, key, int, where)
    if value < 1:
        raise ConfigError(f"config.json: {where}: key {key!r} must be positive, got {value}")
    return value


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int            # size of a query / key head
    vdim: int           # size of a value head
    scale: float        # multiplies q.k
    window: int         # keys a query sees, itself included; 0: every earlier key

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "WindowAttentionConfig":
        heads, kv_heads = _count(raw, "heads", where), _count(raw, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
        mask = raw.get("mask")
        window = _count(mask, "size", where + ".mask") if mask is not None else 0
        return cls(heads, kv_heads, _count(raw, "dim", where), _count(raw, "vdim", where),
                   float(_get(raw, "scale", (int, float), where)), window)

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                                   scale=self.scale)
        if self.window:
            raw["mask"] = {"size": self.window}
        return raw


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]   # one factor per head

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "LightningConfig":
        heads = _count(raw, "heads", where)
        decay = _get(raw, "decay", list, where)
        if len(decay) != heads or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
            raise ConfigError(f"config.json: {where}: 'decay' must give one number per head ({heads})")
        return cls(heads, _count(raw, "dim", where), _count(raw, "vdim", where), tuple(float(d) for d in decay))

    def to_dict(self) -> dict[str, Any]:
        return dict(heads=self.heads, dim=self.dim, vdim=self.vdim, decay=list(self.decay))


@dataclass(frozen=True)
class RoutedExpertsConfig:
    experts: int
    top: int
    ff: int

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "RoutedExpertsConfig":
        kind = raw.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"config.json: {where}: feed-forward kind {kind!r} is not built (only 'moe')")
        router = _get(raw, "router", dict, where)
        experts, top = _count(router, "experts", where + ".router"), _count(router, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}: 'top' ({top}) exceeds 'experts' ({experts})")
        return cls(experts, top, _count(_get(raw, "expert", dict, where), "ff", where + ".expert"))

    def to_dict(self) -> dict[str, Any]:
        return dict(kind="moe", expert=dict(ff=self.ff), router=dict(experts=self.experts, top=self.top))


@dataclass(frozen=True)
class ZisesunLayerConfig:
    type: str                                            # "attention" | "lightning"
    mixer: WindowAttentionConfig | LightningConfig
    mlp: RoutedExpertsConfig | None
    weights_of: int | None                               # layer whose tensors this layer uses

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(type=self.type, mixer=self.mixer.to_dict(),
                                   mlp=self.mlp.to_dict() if self.mlp is not None else None)
        if self.weights_of is not None:
            raw["weights_of"] = self.weights_of
        return raw


MIXERS = {"attention": WindowAttentionConfig, "lightning": LightningConfig}


@dataclass(frozen=True)
class ZisesunConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    streams: int | None                 # None: one plain residual stream, no hyper-connections
    layers: tuple[ZisesunLayerConfig, ...]
    architecture: str = "Zisesun"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ZisesunConfig":
        where = "Zisesun"
        eps = float(_get(_get(raw, "norm", dict, where), "eps", (int, float), where + ".norm"))
        if eps < 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {eps}")
        streams = None if raw.get("streams") is None else _count(raw, "streams", where)
        entries = _get(raw, "layers", list, where)
        if not entries:
            raise ConfigError("config.json: 'layers' is empty")
        layers: list[ZisesunLayerConfig] = []
        for index, entry in enumerate(entries):
            here = f"layers[{index}]"
            kind = _get(entry, "type", str, here)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {here}: mixer type {kind!r} is not built (known: {sorted(MIXERS)})")
            mixer = MIXERS[kind].from_dict(_get(entry, "mixer", dict, here), here + ".mixer")
            mlp = entry.get("mlp")
            mlp = RoutedExpertsConfig.from_dict(mlp, here + ".mlp") if mlp is not None else None
            weights_of = entry.get("weights_of")
            if weights_of is not None:
                if isinstance(weights_of, bool) or not isinstance(weights_of, int) or not 0 <= weights_of < index:
                    raise ConfigError(f"config.json: {here}: 'weights_of' must name an earlier layer, got {weights_of!r}")
                owner = layers[weights_of]
                if owner.weights_of is not None:
                    weights_of = owner.weights_of
                    owner = layers[weights_of]
                if (owner.type, owner.mixer, owner.mlp) != (kind, mixer, mlp):
                    raise ConfigError(f"config.json: {here}: differs from layer {weights_of}, whose weights it uses")
            layers.append(ZisesunLayerConfig(kind, mixer, mlp, weights_of))
        return cls(vocab=_count(raw, "vocab", where), width=_count(raw, "width", where),
                   max_positions=_count(raw, "max_positions", where), norm_eps=eps, streams=streams,
                   layers=tuple(layers), architecture=str(raw.get("architecture", "Zisesun")))

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(architecture=self.architecture, vocab=self.vocab, width=self.width,
                                   max_positions=self.max_positions, norm=dict(eps=self.norm_eps),
                                   layers=[layer.to_dict() for layer in self.layers])
        if self.streams is not None:
            raw["streams"] = self.streams
        return raw
