"""Kedasun configuration: the keys of its config.json.

A small decoder-only family of attention layers of two kinds, each layer a sandwich of four grouped RMS norms::

    architecture   "Kedasun"
    vocab, width
    embedding      {"scale"}
    layers         [{"type": "attention" | "attention_2", "mixer": {...}, "mlp": {...} | null}, ...]
    norm           {"eps", "groups"}

``mixer`` of an ``attention`` layer: heads, kv_heads, dim, vdim, scale, rot {base, dims}, v_mix.
``mixer`` of an ``attention_2`` layer: heads, kv_heads, dim, vdim, scale, conv (taps), mask {size, keep_first}
(absent: every earlier key is visible), v_mix.
``mlp``: kind "dense" {ff, limit}.

No size has a default: a key that the model needs and config.json lacks is an error.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Optional

from .base import ConfigError, ModelConfig

LAYER_TYPES = ("attention", "attention_2")
WHO = "KedasunConfig"


def _need(d: Any, key: str, where: str, kind=(int, float)):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"{WHO}: {where} lacks '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"{WHO}: {where}.{key} has the wrong type: {v!r}")
    return v


def _positive(d: Any, keys, where: str) -> None:
    for k in keys:
        if _need(d, k, where, int) <= 0:
            raise ConfigError(f"{WHO}: {where}.{k} must be positive")


def _check_mixer(kind: str, m: Any, where: str) -> None:
    _positive(m, ("heads", "kv_heads", "dim", "vdim"), where)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{WHO}: {where}.heads must be a multiple of kv_heads")
    if not _need(m, "scale", where) > 0:
        raise ConfigError(f"{WHO}: {where}.scale must be positive")
    if m.get("v_mix") is not None and not isinstance(m["v_mix"], bool):
        raise ConfigError(f"{WHO}: {where}.v_mix must be true or false")
    if kind == "attention":
        rot = m.get("rot")
        if rot is not None:
            dims = _need(rot, "dims", where + ".rot", int)
            if dims < 0 or dims % 2 or dims > m["dim"]:
                raise ConfigError(f"{WHO}: {where}.rot.dims must be even and at most dim")
            if dims and not _need(rot, "base", where + ".rot") > 0:
                raise ConfigError(f"{WHO}: {where}.rot.base must be positive")
        return
    _positive(m, ("conv",), where)
    mask = m.get("mask")
    if mask is not None:
        if _need(mask, "size", where + ".mask", int) < 1:
            raise ConfigError(f"{WHO}: {where}.mask.size must be at least 1")
        keep = mask.get("keep_first")
        if keep is not None and (isinstance(keep, bool) or not isinstance(keep, int) or keep < 0):
            raise ConfigError(f"{WHO}: {where}.mask.keep_first must be a count")


def _check_mlp(mlp: Any, where: str) -> None:
    if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
        raise ConfigError(f"{WHO}: {where}.kind must be 'dense'")
    _positive(mlp, ("ff",), where)
    if not _need(mlp, "limit", where) > 0:
        raise ConfigError(f"{WHO}: {where}.limit must be positive")


@dataclasses.dataclass
class KedasunConfig(ModelConfig):
    architecture: ClassVar[str] = "Kedasun"
    model_types: ClassVar[tuple[str, ...]] = ("kedasun",)

    vocab: int = 0
    width: int = 0
    embedding: Optional[dict] = None
    layers: tuple = ()
    norm: Optional[dict] = None

    def to_dict(self) -> dict[str, Any]:
        out = super().to_dict()
        out["architecture"] = self.architecture
        out["layers"] = list(self.layers)
        return out

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"{WHO}: vocab and width must be positive")
        if not self.layers:
            raise ConfigError(f"{WHO}: 'layers' is empty")
        _need(self.embedding, "scale", "embedding")
        if not _need(self.norm, "eps", "norm") > 0:
            raise ConfigError(f"{WHO}: norm.eps must be positive")
        groups = _need(self.norm, "groups", "norm", int)
        if groups < 1 or self.width % groups:
            raise ConfigError(f"{WHO}: norm.groups must divide width")
        mixed = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
                raise ConfigError(f"{WHO}: {where}.type is {layer.get('type') if isinstance(layer, dict) else layer!r}; "
                                  f"known: {LAYER_TYPES}")
            _check_mixer(layer["type"], layer.get("mixer"), where + ".mixer")
            if layer.get("mlp") is not None:
                _check_mlp(layer["mlp"], where + ".mlp")
            m = layer["mixer"]
            if m.get("v_mix"):
                size = m["kv_heads"] * m["vdim"]
                if mixed is not None and size != mixed:
                    raise ConfigError(f"{WHO}: {where}.mixer mixes values of {size} numbers a token with an earlier "
                                      f"layer's {mixed}")
                mixed = size

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def norm_groups(self) -> int:
        return int(self.norm["groups"])

    @property
    def embedding_scale(self) -> float:
        return float(self.embedding["scale"])

    def first_mixing_layer(self) -> Optional[int]:
        """The first layer whose values are mixed into later layers' (None: no layer mixes)."""
        for i, layer in enumerate(self.layers):
            if layer["mixer"].get("v_mix"):
                return i
        return None
