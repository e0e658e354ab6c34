"""Typed configuration of the Lodalix decoder, read from config.json keys.

A Lodalix model is a list of layers; each has one token mixer and, beside it, an optional dense
feed-forward that reads the same normalised input.  config.json carries:

* ``architecture`` "Lodalix", ``vocab``, ``width``, ``norm.eps``;
* ``layers``: per layer ``type`` ("latent_attention", "latent_attention_2" or "general_delta"),
  ``mixer`` (its sizes and constants) and ``mlp`` (null, or ``kind`` "dense" with ``ff`` and ``limit``).

Latent attention: ``heads``, ``dim`` (plain query/key size of a head), ``rot_dim`` (rotated size),
``vdim``, ``kv_rank``, ``q_rank``, ``scale``, ``rot`` (``base``, ``dims`` and optionally ``scaling``
with ``factor``, ``original``, ``fast``, ``slow``) and, for the second kind, optionally ``kv_from``:
the layer whose cached latent this layer reads instead of making its own.  Generalized delta rule:
``heads``, ``dim``; the width of its low-rank decay projection is a tensor's shape (``decay_rank``
may name it, and is written for random models).

Every size and constant comes from here; this module is the only place that knows the key names.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .model_config import ConfigError
from .zisesun_config import _count, _get


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: tuple[float, float, float, float] | None     # factor, original, fast, slow

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "RotaryConfig":
        dims = _count(raw, "dims", where)
        if dims % 2:
            raise ConfigError(f"config.json: {where}: 'dims' must be even, got {dims}")
        base = float(_get(raw, "base", (int, float), where))
        if base <= 1.0:
            raise ConfigError(f"config.json: {where}: 'base' must be above 1, got {base}")
        scaling = raw.get("scaling")
        if scaling is not None:
            here = where + ".scaling"
            scaling = tuple(float(_get(scaling, key, (int, float), here)) for key in ("factor", "original", "fast", "slow"))
            if scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0:
                raise ConfigError(f"config.json: {here}: factor, original, fast and slow must be positive")
        return cls(base, dims, scaling)

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(base=self.base, dims=self.dims)
        if self.scaling is not None:
            factor, original, fast, slow = self.scaling
            raw["scaling"] = dict(factor=factor, original=int(original) if original == int(original) else original,
                                  fast=fast, slow=slow)
        return raw


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int            # plain (unrotated) query / key size of a head
    rot_dim: int        # rotated query / key size of a head; the key part is shared by all heads
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: RotaryConfig
    kv_from: int | None = None      # layer whose cached latent and rotated key part this layer reads

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "LatentAttentionConfig":
        rot = RotaryConfig.from_dict(_get(raw, "rot", dict, where), where + ".rot")
        rot_dim = _count(raw, "rot_dim", where)
        if rot.dims > rot_dim:
            raise ConfigError(f"config.json: {where}: rot.dims ({rot.dims}) exceeds rot_dim ({rot_dim})")
        kv_from = raw.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or kv_from < 0):
            raise ConfigError(f"config.json: {where}: 'kv_from' must be a layer index, got {kv_from!r}")
        return cls(_count(raw, "heads", where), _count(raw, "dim", where), rot_dim, _count(raw, "vdim", where),
                   _count(raw, "kv_rank", where), _count(raw, "q_rank", where),
                   float(_get(raw, "scale", (int, float), where)), rot, kv_from)

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim,
                                   kv_rank=self.kv_rank, q_rank=self.q_rank, scale=self.scale, rot=self.rot.to_dict())
        if self.kv_from is not None:
            raw["kv_from"] = self.kv_from
        return raw


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    dim: int
    decay_rank: int | None = None   # None: the shape of the stored tensor says

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "DeltaConfig":
        rank = raw.get("decay_rank")
        return cls(_count(raw, "heads", where), _count(raw, "dim", where),
                   None if rank is None else _count(raw, "decay_rank", where))

    def to_dict(self) -> dict[str, Any]:
        raw: dict[str, Any] = dict(heads=self.heads, dim=self.dim)
        if self.decay_rank is not None:
            raw["decay_rank"] = self.decay_rank
        return raw


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "DenseMlpConfig":
        kind = raw.get("kind", "dense")
        if kind != "dense":
            raise ConfigError(f"config.json: {where}: feed-forward kind {kind!r} is not built (only 'dense')")
        limit = float(_get(raw, "limit", (int, float), where))
        if limit <= 0:
            raise ConfigError(f"config.json: {where}: 'limit' must be positive, got {limit}")
        return cls(_count(raw, "ff", where), limit)

    def to_dict(self) -> dict[str, Any]:
        return dict(kind="dense", ff=self.ff, limit=self.limit)


MIXERS = {"latent_attention": LatentAttentionConfig, "latent_attention_2": LatentAttentionConfig,
          "general_delta": DeltaConfig}


@dataclass(frozen=True)
class LodalixLayerConfig:
    type: str
    mixer: LatentAttentionConfig | DeltaConfig
    mlp: DenseMlpConfig | None

    def to_dict(self) -> dict[str, Any]:
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp is not None else None)


@dataclass(frozen=True)
class LodalixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[LodalixLayerConfig, ...]
    architecture: str = "Lodalix"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "LodalixConfig":
        where = "Lodalix"
        eps = float(_get(_get(raw, "norm", dict, where), "eps", (int, float), where + ".norm"))
        if eps < 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {eps}")
        entries = _get(raw, "layers", list, where)
        if not entries:
            raise ConfigError("config.json: 'layers' is empty")
        layers: list[LodalixLayerConfig] = []
        for index, entry in enumerate(entries):
            here = f"layers[{index}]"
            kind = _get(entry, "type", str, here)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {here}: mixer type {kind!r} is not built (known: {sorted(MIXERS)})")
            mixer = MIXERS[kind].from_dict(_get(entry, "mixer", dict, here), here + ".mixer")
            source = getattr(mixer, "kv_from", None)
            if source is not None:
                owner = layers[source] if source < index else None
                if (owner is None or owner.type != kind or owner.mixer.kv_from is not None
                        or (owner.mixer.kv_rank, owner.mixer.rot_dim, owner.mixer.rot)
                        != (mixer.kv_rank, mixer.rot_dim, mixer.rot)):
                    raise ConfigError(
                        f"config.json: {here}: 'kv_from' must name an earlier layer of the same kind that makes "
                        f"its own latent, with the same kv_rank, rot_dim and rotation; got {source}")
            mlp = entry.get("mlp")
            mlp = DenseMlpConfig.from_dict(mlp, here + ".mlp") if mlp is not None else None
            layers.append(LodalixLayerConfig(kind, mixer, mlp))
        return cls(vocab=_count(raw, "vocab", where), width=_count(raw, "width", where), norm_eps=eps,
                   layers=tuple(layers), architecture=str(raw.get("architecture", "Lodalix")))

    def to_dict(self) -> dict[str, Any]:
        return dict(architecture=self.architecture, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                    layers=[layer.to_dict() for layer in self.layers])
