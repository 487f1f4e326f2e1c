"""Typed configuration of a Bigerax decoder, read from its ``config.json``.

The file gives every size and every constant that differs between models of the design, layer by layer::

    {"architecture": "Bigerax", "vocab": V, "width": D,
     "embedding": {"bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "norm": {"eps": e, "groups": g},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                                                "rot": {"base", "dims"}, "v_mix"},
                 "mlp": {"kind": "dense", "ff": F} | null},
                {"type": "mingru", "mixer": {"width": W}, "mlp": ...}, ...]}

Required keys fail with the key's path; keys that may be absent (``mask``, ``rot``, ``v_mix``, ``mlp``) mean "the
layer has none".  Same "required key throws" manner as the reference's config readers (src/model/LlmConfig.cpp:64-93).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError

ARCHITECTURE = "Bigerax"


@dataclass(frozen=True)
class AttentionLayer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int            # 0: every earlier token
    rot_dims: int          # 0: no rotation
    rot_base: float
    v_mix: bool


@dataclass(frozen=True)
class MinGRULayer:
    width: int


@dataclass(frozen=True)
class DenseFeedForward:
    ff: int


@dataclass(frozen=True)
class BigeraxLayer:
    type: str                               # "attention" or "mingru"
    mixer: Any                              # AttentionLayer or MinGRULayer
    mlp: Optional[DenseFeedForward]


@dataclass(frozen=True)
class BigeraxConfig:
    architecture: str
    vocab: int
    width: int
    buckets: int
    mul_prev: int
    mul_cur: int
    norm_eps: float
    norm_groups: int
    layers: Tuple[BigeraxLayer, ...]
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()


class _At:
    """A JSON object with the path to it, for messages."""

    def __init__(self, obj: Any, path: str, where: str):
        if not isinstance(obj, dict):
            raise ConfigError(f"{where}: '{path}' is not an object")
        self.obj, self.path, self.where = obj, path, where

    def _name(self, key: str) -> str:
        return f"{self.path}.{key}" if self.path else key

    def need(self, key: str) -> Any:
        if key not in self.obj or self.obj[key] is None:
            raise ConfigError(f"{self.where}: missing required key '{self._name(key)}'")
        return self.obj[key]

    def integer(self, key: str, minimum: Optional[int] = 1) -> int:
        v = self.need(key)
        if isinstance(v, bool) or not isinstance(v, int) or (minimum is not None and v < minimum):
            raise ConfigError(f"{self.where}: '{self._name(key)}' must be an integer" + (f" >= {minimum}" if minimum is not None else "") + f", got {v!r}")
        return v

    def number(self, key: str) -> float:
        v = self.need(key)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: '{self._name(key)}' must be a number, got {v!r}")
        return float(v)

    def child(self, key: str) -> "_At":
        return _At(self.need(key), self._name(key), self.where)

    def maybe(self, key: str) -> Optional["_At"]:
        return _At(self.obj[key], self._name(key), self.where) if self.obj.get(key) is not None else None


def parse_bigerax_config(obj: Dict[str, Any], where: str = "config.json") -> BigeraxConfig:
    top = _At(obj, "", where)
    width = top.integer("width")
    big = top.child("embedding").child("bigram")
    norm = top.child("norm")
    groups = norm.integer("groups")
    if width % groups:
        raise ConfigError(f"{where}: norm.groups = {groups} does not divide width = {width}")
    raw_layers = top.need("layers")
    if not isinstance(raw_layers, list) or not raw_layers:
        raise ConfigError(f"{where}: 'layers' must be a non-empty list")
    layers = []
    for i, raw in enumerate(raw_layers):
        at = _At(raw, f"layers[{i}]", where)
        kind = at.need("type")
        m = at.child("mixer")
        if kind == "attention":
            heads, kv = m.integer("heads"), m.integer("kv_heads")
            if heads % kv:
                raise ConfigError(f"{where}: layers[{i}].mixer.heads = {heads} is not a multiple of kv_heads = {kv}")
            dim = m.integer("dim")
            mask, rot = m.maybe("mask"), m.maybe("rot")
            rot_dims = rot.integer("dims", 0) if rot is not None else 0
            if rot_dims % 2 or rot_dims > dim:
                raise ConfigError(f"{where}: layers[{i}].mixer.rot.dims = {rot_dims} must be even and at most dim = {dim}")
            mixer = AttentionLayer(heads=heads, kv_heads=kv, dim=dim, vdim=m.integer("vdim"), scale=m.number("scale"),
                                   window=mask.integer("size") if mask is not None else 0, rot_dims=rot_dims,
                                   rot_base=rot.number("base") if rot is not None and rot_dims else 1.0, v_mix=bool(m.obj.get("v_mix", False)))
        elif kind == "mingru":
            mixer = MinGRULayer(width=m.integer("width"))
        else:
            raise ConfigError(f"{where}: layers[{i}].type = {kind!r} is not one of 'attention', 'mingru'")
        mlp_at = at.maybe("mlp")
        mlp = None
        if mlp_at is not None:
            if mlp_at.need("kind") != "dense":
                raise ConfigError(f"{where}: layers[{i}].mlp.kind = {mlp_at.obj['kind']!r} is not 'dense'")
            mlp = DenseFeedForward(ff=mlp_at.integer("ff"))
        layers.append(BigeraxLayer(type=kind, mixer=mixer, mlp=mlp))
    eos = obj.get("eos_token_id")
    eos_ids = tuple(eos) if isinstance(eos, list) else ((eos,) if isinstance(eos, int) else ())
    max_pos = obj.get("max_positions")
    return BigeraxConfig(
        architecture=str(obj.get("architecture", ARCHITECTURE)), vocab=top.integer("vocab"), width=width,
        buckets=big.integer("buckets"), mul_prev=big.integer("mul_prev", None), mul_cur=big.integer("mul_cur", None),
        norm_eps=norm.number("eps"), norm_groups=groups, layers=tuple(layers),
        max_positions=int(max_pos) if isinstance(max_pos, int) and max_pos > 0 else 1 << 20, eos_token_ids=eos_ids)
