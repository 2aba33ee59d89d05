"""Typed configuration of Bisudra, read from its own config.json keys.

A Bisudra folder names itself with `"architecture": "Bisudra"`.  `layers` lists the layers; each entry has a `type` (which mixer:
`attention`, a differential attention), the mixer's sizes and constants under `mixer` and its feed-forward under `mlp` (null: none;
`kind` `dense` or `moe`).  `canon.taps`, `token_side.dim`, `norm.eps`, `vocab` and `width` are model-wide.  Every size and constant that
can differ between models is read here and nowhere else.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .errors import InvalidConfig
from .fasesun import _integer, _number, _object
from .metadata import metadata_from_json

ARCHITECTURE = "Bisudra"
MODEL_TYPE = "bisudra"
MIXER_TYPES = ("attention",)


@dataclass(frozen=True)
class DifferentialAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    window: int
    rot_base: float
    rot_dims: int
    type: str = "attention"


@dataclass(frozen=True)
class DenseConfig:
    ff: int
    kind: str = "dense"


@dataclass(frozen=True)
class MoEConfig:
    experts: int
    top: int
    expert_ff: int
    kind: str = "moe"


@dataclass(frozen=True)
class LayerConfig:
    mixer: DifferentialAttentionConfig
    mlp: Optional[object]


def _mixer(raw: dict, where: str) -> DifferentialAttentionConfig:
    heads, kv_heads, dim, vdim = (_integer(raw, key, where) for key in ("heads", "kv_heads", "dim", "vdim"))
    if heads % kv_heads:
        raise InvalidConfig(f"config.json: {where}heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    rot = _object(raw, "rot", where)
    rot_dims = _integer(rot, "dims", where + "rot.", 0)
    if rot_dims % 2 or rot_dims > dim:
        raise InvalidConfig(f"config.json: {where}rot.dims must be even and at most dim ({dim}), found {rot_dims}")
    diff = _number(raw, "diff", where, positive=False)
    return DifferentialAttentionConfig(heads, kv_heads, dim, vdim, _number(raw, "scale", where), diff,
                                       _integer(_object(raw, "mask", where), "size", where + "mask."), _number(rot, "base", where + "rot."), rot_dims)


def _mlp(raw, where: str):
    if raw is None:
        return None
    if not isinstance(raw, dict) or raw.get("kind") not in ("dense", "moe"):
        raise InvalidConfig(f"config.json: {where} must be null or an object of kind 'dense' or 'moe'")
    if raw["kind"] == "dense":
        return DenseConfig(_integer(raw, "ff", where + "."))
    router = _object(raw, "router", where + ".")
    experts, top = _integer(router, "experts", where + ".router."), _integer(router, "top", where + ".router.")
    if top > experts:
        raise InvalidConfig(f"config.json: {where}.router.top ({top}) exceeds router.experts ({experts})")
    return MoEConfig(experts, top, _integer(_object(raw, "expert", where + "."), "ff", where + ".expert."))


@dataclass(frozen=True)
class BisudraConfig:
    vocab: int
    width: int
    eps: float
    taps: int
    side_dim: int
    layers: Tuple[LayerConfig, ...]
    declared_dtype: Optional[str] = None

    architecture = ARCHITECTURE
    model_type = MODEL_TYPE

    @classmethod
    def from_json(cls, raw: dict) -> "BisudraConfig":
        metadata = metadata_from_json(raw)
        if metadata.architecture != ARCHITECTURE:
            raise InvalidConfig(f"expected {ARCHITECTURE}, found {metadata.architecture}")
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise InvalidConfig("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for index, entry in enumerate(listed):
            where = f"layers[{index}]."
            if not isinstance(entry, dict) or entry.get("type") not in MIXER_TYPES:
                raise InvalidConfig(f"config.json: {where}type must be one of {', '.join(MIXER_TYPES)}")
            layers.append(LayerConfig(_mixer(_object(entry, "mixer", where), where + "mixer."), _mlp(entry.get("mlp"), where + "mlp")))
        return cls(vocab=_integer(raw, "vocab", ""), width=_integer(raw, "width", ""), eps=_number(_object(raw, "norm", ""), "eps", "norm."),
                   taps=_integer(_object(raw, "canon", ""), "taps", "canon."), side_dim=_integer(_object(raw, "token_side", ""), "dim", "token_side."),
                   layers=tuple(layers), declared_dtype=metadata.declared_dtype)
