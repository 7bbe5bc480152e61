"""Ritirax configuration: the keys of its config.json.

A small decoder-only family that lists its layers one by one and mixes three kinds of token mixing::

    architecture   "Ritirax"
    vocab, width
    embedding      {"scale"}         the looked-up row is multiplied by it
    layers         [{"type": "attention" | "latent_attention" | "lightning", "mixer": {...}, "mlp": {...} | null}, ...]
    norm           {"eps"}

``mixer`` of an ``attention`` layer: heads, kv_heads, dim, vdim, scale, softcap (absent or 0: no cap), bias_max (the
distance at which the learned distance bias reaches its last row; the table's rows are the shape of the checkpoint's
tensor, and the optional key bias_rows only says how many a model made at random gets).
``mixer`` of a ``latent_attention`` layer: heads, dim (unrotated query/key size per head), rot_dim (rotated), vdim,
kv_rank, scale, rot {base, dims, scaling {factor, original, fast, slow} | absent}.
``mixer`` of a ``lightning`` layer: heads, dim, vdim, decay (one number per head).
``mlp``: kind "dense" {ff}, or kind "moe" {expert {ff}, router {experts, top, scale, groups {count, keep} | absent},
shared {ff} | absent}.

No size has a default: a key that the model needs and config.json lacks is an error.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Optional

from .base import ConfigError, ModelConfig

LAYER_TYPES = ("attention", "latent_attention", "lightning")
MLP_KINDS = ("dense", "moe")
WHO = "RitiraxConfig"


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


def _check_attention(m: Any, where: str) -> None:
    _positive(m, ("heads", "kv_heads", "dim", "vdim"), where)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{WHO}: {where}.heads must be a multiple of kv_heads")
    if not _need(m, "scale", where) > 0:
        raise ConfigError(f"{WHO}: {where}.scale must be positive")
    if m.get("softcap") is not None and _need(m, "softcap", where) < 0:
        raise ConfigError(f"{WHO}: {where}.softcap cannot be negative")
    if not _need(m, "bias_max", where) > 1:
        raise ConfigError(f"{WHO}: {where}.bias_max must be beyond 1")


def _check_latent(m: Any, where: str) -> None:
    _positive(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank"), where)
    if not _need(m, "scale", where) > 0:
        raise ConfigError(f"{WHO}: {where}.scale must be positive")
    rot = m.get("rot")
    dims = _need(rot, "dims", where + ".rot", int)
    if dims <= 0 or dims % 2 or dims > m["rot_dim"]:
        raise ConfigError(f"{WHO}: {where}.rot.dims must be even, positive and at most rot_dim")
    if not _need(rot, "base", where + ".rot") > 1:
        raise ConfigError(f"{WHO}: {where}.rot.base must be beyond 1")
    sc = rot.get("scaling")
    if sc is not None:
        for k in ("factor", "original", "fast", "slow"):
            if not _need(sc, k, where + ".rot.scaling") > 0:
                raise ConfigError(f"{WHO}: {where}.rot.scaling.{k} must be positive")


def _check_lightning(m: Any, where: str) -> None:
    _positive(m, ("heads", "dim", "vdim"), where)
    decay = m.get("decay")
    if not isinstance(decay, (list, tuple)) or len(decay) != m["heads"]:
        raise ConfigError(f"{WHO}: {where}.decay must list one number per head")
    for d in decay:
        if isinstance(d, bool) or not isinstance(d, (int, float)) or not 0 <= d <= 1:
            raise ConfigError(f"{WHO}: {where}.decay holds {d!r}; every decay lies between 0 and 1")


def _check_mlp(mlp: Any, where: str) -> None:
    if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
        raise ConfigError(f"{WHO}: {where}.kind must be one of {MLP_KINDS}")
    if mlp["kind"] == "dense":
        _positive(mlp, ("ff",), where)
        return
    _positive(mlp.get("expert"), ("ff",), where + ".expert")
    router = mlp.get("router")
    _positive(router, ("experts", "top"), where + ".router")
    n, top = router["experts"], router["top"]
    if router.get("scale") is not None:
        _need(router, "scale", where + ".router")
    count, keep = 1, 1
    if router.get("groups") is not None:
        _positive(router["groups"], ("count", "keep"), where + ".router.groups")
        count, keep = router["groups"]["count"], router["groups"]["keep"]
    if n % count or keep > count:
        raise ConfigError(f"{WHO}: {where}.router.groups: count must divide experts, and keep cannot exceed count")
    if top > keep * (n // count):
        raise ConfigError(f"{WHO}: {where}.router.top exceeds the experts of the groups that stay open")
    if mlp.get("shared") is not None:
        _positive(mlp["shared"], ("ff",), where + ".shared")


_CHECKS = {"attention": _check_attention, "latent_attention": _check_latent, "lightning": _check_lightning}


@dataclasses.dataclass
class RitiraxConfig(ModelConfig):
    architecture: ClassVar[str] = "Ritirax"
    model_types: ClassVar[tuple[str, ...]] = ("ritirax",)

    vocab: int = 0
    width: int = 0
    layers: tuple = ()
    norm: Optional[dict] = None
    embedding: Optional[dict] = None

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
        if not _need(self.norm, "eps", "norm") > 0:
            raise ConfigError(f"{WHO}: norm.eps must be positive")
        _need(self.embedding, "scale", "embedding")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
                raise ConfigError(f"{WHO}: {where}.type is {layer.get('type') if isinstance(layer, dict) else layer!r}; "
                                  f"known: {LAYER_TYPES}")
            _CHECKS[layer["type"]](layer.get("mixer"), where + ".mixer")
            if layer.get("mlp") is not None:
                _check_mlp(layer["mlp"], where + ".mlp")

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def embedding_scale(self) -> float:
        return float(self.embedding["scale"])
