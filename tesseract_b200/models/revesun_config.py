"""Typed configuration of the ``Revesun`` architecture, read from ``config.json``.

``config.json`` names the architecture under ``architecture`` and gives ``width`` (the residual stream), ``vocab``,
``norm`` (``eps`` and ``groups`` of every norm) and ``layers``: a list whose entries each give ``type`` (which mixer),
``mixer`` (that mixer's sizes and constants) and ``mlp`` (``{"kind": "dense", "ff": n}`` or null).  Layers may differ
from one another in every number and come in any order.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..config.reading import ConfigError, require as _require


@dataclass(frozen=True)
class RevesunAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    block: int                   # mask.size: positions are cut into blocks of this many
    rot_dims: int
    rot_base: float
    scale: float

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "RevesunAttention":
        mask = _require(data, "mask", dict, where)
        rot = _require(data, "rot", dict, where)
        out = cls(heads=_require(data, "heads", int, where), kv_heads=_require(data, "kv_heads", int, where),
                  dim=_require(data, "dim", int, where), vdim=_require(data, "vdim", int, where),
                  conv=_require(data, "conv", int, where), block=_require(mask, "size", int, where + ".mask"),
                  rot_dims=_require(rot, "dims", int, where + ".rot"),
                  rot_base=float(_require(rot, "base", (int, float), where + ".rot")),
                  scale=float(_require(data, "scale", (int, float), where)))
        if out.heads <= 0 or out.kv_heads <= 0 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}: heads must be a positive multiple of kv_heads")
        if out.dim <= 0 or out.vdim <= 0:
            raise ConfigError(f"{where}: dim and vdim must be positive")
        if out.conv < 1:
            raise ConfigError(f"{where}: conv (the number of taps) must be at least 1")
        if out.block < 1:
            raise ConfigError(f"{where}: mask.size must be positive")
        if out.rot_dims < 0 or out.rot_dims % 2 or out.rot_dims > out.dim:
            raise ConfigError(f"{where}: rot.dims must be even and at most dim")
        if not (out.rot_base > 0 and math.isfinite(out.rot_base)) or not math.isfinite(out.scale):
            raise ConfigError(f"{where}: rot.base must be positive and scale finite")
        return out


@dataclass(frozen=True)
class RevesunMinGRU:
    width: int

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "RevesunMinGRU":
        out = cls(width=_require(data, "width", int, where))
        if out.width <= 0:
            raise ConfigError(f"{where}: width must be positive")
        return out


@dataclass(frozen=True)
class RevesunLayer:
    type: str
    mixer: Union[RevesunAttention, RevesunMinGRU]
    ff: Optional[int]            # None: the layer has no feed-forward


_MIXERS = {"attention": RevesunAttention, "mingru": RevesunMinGRU}


@dataclass(frozen=True)
class RevesunConfig:
    width: int
    vocab: int
    norm_eps: float
    norm_groups: int
    layers: Tuple[RevesunLayer, ...]

    ARCHITECTURE = "Revesun"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "RevesunConfig":
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
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp: only kind 'dense' is known")
                ff = _require(mlp, "ff", int, where + ".mlp")
                if ff <= 0:
                    raise ConfigError(f"{where}.mlp: ff must be positive")
            layers.append(RevesunLayer(kind, mixer, ff))
        cfg = cls(width=_require(data, "width", int), vocab=_require(data, "vocab", int),
                  norm_eps=float(_require(norm, "eps", (int, float), "norm")),
                  norm_groups=_require(norm, "groups", int, "norm"), layers=tuple(layers))
        if cfg.width <= 0 or cfg.vocab <= 0 or not cfg.layers:
            raise ConfigError("width and vocab must be positive and layers not empty")
        if cfg.norm_groups < 1 or cfg.width % cfg.norm_groups:
            raise ConfigError("norm.groups must divide width")
        if not (cfg.norm_eps > 0 and math.isfinite(cfg.norm_eps)):
            raise ConfigError("norm.eps must be finite and positive")
        return cfg
