"""Typed configuration of a Domelix decoder, read from its ``config.json``.

The file gives every size and every constant that differs between models of the design, layer by layer::

    {"architecture": "Domelix", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "parallel", "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "bias_max", "bias_rows"?},
                                               "right": {"heads", "dim", "vdim", "decay": [one per head]}}, "mlp": ...},
                {"type": "delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": ...},
                {"type": "retention", "mixer": {"heads", "dim", "vdim", "decay": [one per head], "rot": {"base", "dims"}}, "mlp": ...}]}

with ``mlp`` either null or ``{"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k, "groups": {"count", "keep"}}}``.
Required keys fail with the key's path; ``rot``, ``groups`` and ``mlp`` may be absent and mean "the layer has none";
``bias_rows`` (the rows of the left mixer's distance table) may be absent: the checkpoint's table then decides, and only the
random-weights mode needs the key.
Same "required key throws" manner as the reference's config readers (src/model/LlmConfig.cpp:64-93).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .bigerax_config import _At
from .model_config import ConfigError

ARCHITECTURE = "Domelix"


@dataclass(frozen=True)
class BiasedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: float
    bias_rows: Optional[int] = None      # rows of the distance table; None: as many as the checkpoint's table has


@dataclass(frozen=True)
class DecayedState:
    """Linear attention with one constant decay per head; ``rot_dims`` 0: no rotation."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_dims: int = 0
    rot_base: float = 1.0


@dataclass(frozen=True)
class ParallelMixer:
    left: BiasedAttention
    right: DecayedState


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class ExpertsFeedForward:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int


@dataclass(frozen=True)
class DomelixLayer:
    type: str                               # "parallel", "delta" or "retention"
    mixer: Any
    mlp: Optional[ExpertsFeedForward]


@dataclass(frozen=True)
class DomelixConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[DomelixLayer, ...]
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()


def _decay(at: _At, heads: int) -> Tuple[float, ...]:
    raw = at.need("decay")
    if not isinstance(raw, list) or len(raw) != heads or any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in raw):
        raise ConfigError(f"{at.where}: '{at._name('decay')}' must be a list of {heads} numbers, one per head")
    return tuple(float(x) for x in raw)


def _decayed(at: _At, i: int) -> DecayedState:
    heads, dim = at.integer("heads"), at.integer("dim")
    rot = at.maybe("rot")
    rot_dims = rot.integer("dims", 0) if rot is not None else 0
    if rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"{at.where}: '{at._name('rot.dims')}' = {rot_dims} must be even and at most dim = {dim}")
    return DecayedState(heads=heads, dim=dim, vdim=at.integer("vdim"), decay=_decay(at, heads), rot_dims=rot_dims,
                        rot_base=rot.number("base") if rot is not None and rot_dims else 1.0)


def _grouped(at: _At, what: str) -> Tuple[int, int]:
    heads, kv = at.integer("heads"), at.integer("kv_heads")
    if heads % kv:
        raise ConfigError(f"{at.where}: '{at._name('heads')}' = {heads} is not a multiple of kv_heads = {kv}")
    return heads, kv


def parse_domelix_config(obj: Dict[str, Any], where: str = "config.json") -> DomelixConfig:
    top = _At(obj, "", where)
    width = top.integer("width")
    raw_layers = top.need("layers")
    if not isinstance(raw_layers, list) or not raw_layers:
        raise ConfigError(f"{where}: 'layers' must be a non-empty list")
    layers = []
    for i, raw in enumerate(raw_layers):
        at = _At(raw, f"layers[{i}]", where)
        kind = at.need("type")
        m = at.child("mixer")
        if kind == "parallel":
            left, right = m.child("left"), m.child("right")
            heads, kv = _grouped(left, "left")
            mixer = ParallelMixer(
                left=BiasedAttention(heads=heads, kv_heads=kv, dim=left.integer("dim"), vdim=left.integer("vdim"), scale=left.number("scale"),
                                     bias_max=left.number("bias_max"),
                                     bias_rows=left.integer("bias_rows", 2) if left.obj.get("bias_rows") is not None else None),
                right=_decayed(right, i))
        elif kind == "delta":
            heads, kv = _grouped(m, "mixer")
            mixer = DeltaMixer(heads=heads, kv_heads=kv, dim=m.integer("dim"), vdim=m.integer("vdim"), conv=m.integer("conv"))
        elif kind == "retention":
            mixer = _decayed(m, i)
        else:
            raise ConfigError(f"{where}: layers[{i}].type = {kind!r} is not one of 'parallel', 'delta', 'retention'")
        mlp_at = at.maybe("mlp")
        mlp = None
        if mlp_at is not None:
            if mlp_at.need("kind") != "moe":
                raise ConfigError(f"{where}: layers[{i}].mlp.kind = {mlp_at.obj['kind']!r} is not 'moe'")
            router = mlp_at.child("router")
            experts, chosen = router.integer("experts"), router.integer("top")
            groups = router.maybe("groups")
            count, keep = (groups.integer("count"), groups.integer("keep")) if groups is not None else (1, 1)
            if experts % count or keep > count or chosen > keep * (experts // count):
                raise ConfigError(f"{where}: layers[{i}].mlp.router: {experts} experts in {count} groups, {keep} kept, {chosen} chosen do not fit")
            mlp = ExpertsFeedForward(ff=mlp_at.child("expert").integer("ff"), experts=experts, top=chosen, groups=count, keep=keep)
        layers.append(DomelixLayer(type=kind, mixer=mixer, mlp=mlp))
    eos = obj.get("eos_token_id")
    eos_ids = tuple(eos) if isinstance(eos, list) else ((eos,) if isinstance(eos, int) else ())
    max_pos = obj.get("max_positions")
    return DomelixConfig(architecture=str(obj.get("architecture", ARCHITECTURE)), vocab=top.integer("vocab"), width=width,
                         norm_eps=top.child("norm").number("eps"), layers=tuple(layers),
                         max_positions=int(max_pos) if isinstance(max_pos, int) and max_pos > 0 else 1 << 20, eos_token_ids=eos_ids)
