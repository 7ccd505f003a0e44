"""Typed configuration of the ``Pekodra`` architecture, read from ``config.json``.

``config.json`` names the architecture under ``architecture`` and gives ``width`` (the residual stream), ``vocab``,
``norm.eps``, ``embedding.scale``, ``logit_scale``, ``layers`` and, optionally, ``loop``.  A layer entry gives ``type``
(which mixer; ``attention`` is the one this design has), ``mixer`` (its sizes and constants) and ``mlp``: null, a dense
gated feed-forward (``{"kind": "dense", "ff": n}``) or routed experts (``{"kind": "moe", "router": {"experts", "top"},
"expert": {"ff"}, "shared": {"ff"} or absent}``).  ``loop`` (``start``, ``stop``, ``times``) makes layers ``start`` to
``stop - 1`` run ``times`` times in a row with the same weights.  Layers may differ from one another in every number.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..config.reading import ConfigError, require as _require

_NUMBER = (int, float)


def _positive(value, what: str):
    if not (value > 0 and math.isfinite(value)):
        raise ConfigError(f"{what} must be positive and finite")
    return value


@dataclass(frozen=True)
class PekodraRotation:
    dims: int
    base: float
    # (factor, original, fast, slow) of a stretched context, or None
    scaling: Optional[Tuple[Tuple[str, float], ...]]

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], dim: int, where: str) -> "PekodraRotation":
        dims = _require(data, "dims", int, where)
        base = float(_require(data, "base", _NUMBER, where))
        if dims < 0 or dims % 2 or dims > dim:
            raise ConfigError(f"{where}: dims must be even and at most the head's dim")
        if not (base > 0 and math.isfinite(base)) or base == 1.0:
            raise ConfigError(f"{where}: base must be positive, finite and not 1")
        scaling = data.get("scaling")
        frozen = None
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"{where}.scaling must be an object or null")
            frozen = tuple((key, float(_positive(_require(scaling, key, _NUMBER, where + ".scaling"),
                                                 f"{where}.scaling.{key}")))
                           for key in ("factor", "fast", "original", "slow"))
        return cls(dims, base, frozen)


@dataclass(frozen=True)
class PekodraAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: Optional[int]        # mask.size: a row sees itself and the size - 1 positions before it; None: all
    rotation: Optional[PekodraRotation]
    scale: float

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "PekodraAttention":
        heads, kv_heads = _require(data, "heads", int, where), _require(data, "kv_heads", int, where)
        dim, vdim = _require(data, "dim", int, where), _require(data, "vdim", int, where)
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ConfigError(f"{where}: heads must be a positive multiple of kv_heads")
        if dim <= 0 or vdim <= 0:
            raise ConfigError(f"{where}: dim and vdim must be positive")
        window = None
        if data.get("mask") is not None:
            window = _require(_require(data, "mask", dict, where), "size", int, where + ".mask")
            if window < 1:
                raise ConfigError(f"{where}: mask.size must be positive")
        rotation = None
        if data.get("rot") is not None:
            rotation = PekodraRotation.from_dict(_require(data, "rot", dict, where), dim, where + ".rot")
        scale = float(_require(data, "scale", _NUMBER, where))
        if not math.isfinite(scale):
            raise ConfigError(f"{where}: scale must be finite")
        return cls(heads, kv_heads, dim, vdim, window, rotation, scale)


@dataclass(frozen=True)
class PekodraDense:
    ff: int


@dataclass(frozen=True)
class PekodraExperts:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int]     # None: no shared expert


def _read_mlp(mlp: Any, where: str) -> Union[None, PekodraDense, PekodraExperts]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"{where} must be an object or null")
    kind = _require(mlp, "kind", str, where)
    if kind == "dense":
        ff = _require(mlp, "ff", int, where)
        if ff <= 0:
            raise ConfigError(f"{where}: ff must be positive")
        return PekodraDense(ff)
    if kind == "moe":
        router = _require(mlp, "router", dict, where)
        experts, top = _require(router, "experts", int, where + ".router"), _require(router, "top", int, where + ".router")
        ff = _require(_require(mlp, "expert", dict, where), "ff", int, where + ".expert")
        shared = mlp.get("shared")
        shared_ff = None
        if shared is not None:
            shared_ff = _require(_require(mlp, "shared", dict, where), "ff", int, where + ".shared")
            if shared_ff <= 0:
                raise ConfigError(f"{where}.shared: ff must be positive")
        if experts <= 0 or not 1 <= top <= experts or ff <= 0:
            raise ConfigError(f"{where}: needs experts > 0, 1 <= top <= experts and expert.ff > 0")
        return PekodraExperts(experts, top, ff, shared_ff)
    raise ConfigError(f"{where}: unknown kind '{kind}' (known: dense, moe)")


@dataclass(frozen=True)
class PekodraLayer:
    type: str
    mixer: PekodraAttention
    mlp: Union[None, PekodraDense, PekodraExperts]


@dataclass(frozen=True)
class PekodraLoop:
    start: int
    stop: int
    times: int


_MIXERS = {"attention": PekodraAttention}


@dataclass(frozen=True)
class PekodraConfig:
    width: int
    vocab: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: Tuple[PekodraLayer, ...]
    loop: Optional[PekodraLoop]

    ARCHITECTURE = "Pekodra"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "PekodraConfig":
        norm = _require(data, "norm", dict)
        layers = []
        for index, entry in enumerate(_require(data, "layers", list)):
            where = f"layers[{index}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where} must be an object")
            kind = _require(entry, "type", str, where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}: unknown type '{kind}' (known: {sorted(_MIXERS)})")
            mixer = _MIXERS[kind].from_dict(_require(entry, "mixer", dict, where), where + ".mixer")
            layers.append(PekodraLayer(kind, mixer, _read_mlp(entry.get("mlp"), where + ".mlp")))
        loop = None
        if data.get("loop") is not None:
            raw = _require(data, "loop", dict)
            loop = PekodraLoop(_require(raw, "start", int, "loop"), _require(raw, "stop", int, "loop"),
                               _require(raw, "times", int, "loop"))
            if not (0 <= loop.start <= loop.stop <= len(layers)) or loop.times < 1:
                raise ConfigError("loop: needs 0 <= start <= stop <= number of layers and times >= 1")
        embedding = data.get("embedding")
        embedding_scale = 1.0 if embedding is None else float(_require(_require(data, "embedding", dict), "scale",
                                                                       _NUMBER, "embedding"))
        logit_scale = 1.0 if data.get("logit_scale") is None else float(_require(data, "logit_scale", _NUMBER))
        cfg = cls(width=_require(data, "width", int), vocab=_require(data, "vocab", int),
                  norm_eps=float(_require(norm, "eps", _NUMBER, "norm")), embedding_scale=embedding_scale,
                  logit_scale=logit_scale, layers=tuple(layers), loop=loop)
        if cfg.width <= 0 or cfg.vocab <= 0 or not cfg.layers:
            raise ConfigError("width and vocab must be positive and layers not empty")
        if not (cfg.norm_eps > 0 and math.isfinite(cfg.norm_eps)):
            raise ConfigError("norm.eps must be finite and positive")
        if not (math.isfinite(cfg.embedding_scale) and math.isfinite(cfg.logit_scale)):
            raise ConfigError("embedding.scale and logit_scale must be finite")
        return cfg

    def run_order(self) -> Tuple[Tuple[int, bool], ...]:
        """``(layer, starts a walk)`` in the order the layers run: the looped run ``times`` times, each walk's first
        layer marked."""
        count = len(self.layers)
        if self.loop is None:
            return tuple((i, False) for i in range(count))
        order = [(i, False) for i in range(self.loop.start)]
        for _ in range(self.loop.times):
            order += [(i, i == self.loop.start) for i in range(self.loop.start, self.loop.stop)]
        return tuple(order + [(i, False) for i in range(self.loop.stop, count)])
