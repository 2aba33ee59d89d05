"""Typed configuration of Fasesun, read from its own config.json keys.

A Fasesun folder names itself with `"architecture": "Fasesun"`.  `layers` lists the layers; each entry has a `type`
(which mixer: `latent_attention`, `mlstm` or `lightning`), the mixer's sizes under `mixer` and its feed-forward under
`mlp` (null: none).  `loop` makes the layers `start .. stop-1` run `times` times in a row with the same weights.
`norm.eps`, `vocab` and `width` are model-wide.  Every size and constant that can differ between models is read here
and nowhere else.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

from .errors import InvalidConfig
from .metadata import metadata_from_json

ARCHITECTURE = "Fasesun"
MODEL_TYPE = "fasesun"
MIXER_TYPES = ("latent_attention", "mlstm", "lightning")


def _object(raw, key: str, where: str) -> dict:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise InvalidConfig(f"config.json: {where}{key!r} must be an object")
    return value


def _integer(raw: dict, key: str, where: str, minimum: int = 1) -> int:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value < minimum:
        raise InvalidConfig(f"config.json: {where}{key!r} must be an integer of at least {minimum}, found {value!r}")
    return value


def _number(raw: dict, key: str, where: str, positive: bool = True) -> float:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or (positive and value <= 0):
        raise InvalidConfig(f"config.json: {where}{key!r} must be a finite {'positive ' if positive else ''}number, found {value!r}")
    return float(value)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    type: str = "latent_attention"


@dataclass(frozen=True)
class MLSTMConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float
    type: str = "mlstm"


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    type: str = "lightning"


@dataclass(frozen=True)
class MoEConfig:
    experts: int
    top: int
    expert_ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class LayerConfig:
    mixer: object
    mlp: Optional[MoEConfig]


def _mixer(kind: str, raw: dict, where: str):
    heads, dim, vdim = (_integer(raw, key, where) for key in ("heads", "dim", "vdim"))
    if kind == "latent_attention":
        rot = _object(raw, "rot", where)
        rot_dim = _integer(raw, "rot_dim", where)
        rot_dims = _integer(rot, "dims", where + "rot.")
        if rot_dims % 2 or rot_dims > rot_dim:
            raise InvalidConfig(f"config.json: {where}rot.dims must be even and at most rot_dim ({rot_dim}), found {rot_dims}")
        return LatentAttentionConfig(heads, dim, rot_dim, vdim, _integer(raw, "q_rank", where), _integer(raw, "kv_rank", where),
                                     _number(raw, "scale", where), _number(rot, "base", where + "rot."), rot_dims)
    if kind == "mlstm":
        return MLSTMConfig(heads, dim, vdim, _number(raw, "gate_cap", where))
    decay = raw.get("decay")
    if not isinstance(decay, list) or len(decay) != heads:
        raise InvalidConfig(f"config.json: {where}'decay' must list one number for each of the {heads} heads")
    return LightningConfig(heads, dim, vdim, tuple(_number({"decay": value}, "decay", where) for value in decay))


def _mlp(raw: Optional[dict], where: str) -> Optional[MoEConfig]:
    if raw is None:
        return None
    if not isinstance(raw, dict) or raw.get("kind") != "moe":
        raise InvalidConfig(f"config.json: {where} must be null or an object of kind 'moe'")
    router = _object(raw, "router", where)
    experts, top = _integer(router, "experts", where + "router."), _integer(router, "top", where + "router.")
    if top > experts:
        raise InvalidConfig(f"config.json: {where}router.top ({top}) exceeds router.experts ({experts})")
    shared = raw.get("shared")
    return MoEConfig(experts, top, _integer(_object(raw, "expert", where), "ff", where + "expert."),
                     None if shared is None else _integer(shared, "ff", where + "shared."))


@dataclass(frozen=True)
class FasesunConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[LayerConfig, ...]
    loop_start: int
    loop_stop: int
    loop_times: int
    declared_dtype: Optional[str] = None

    architecture = ARCHITECTURE
    model_type = MODEL_TYPE

    def layer_runs(self) -> Tuple[int, ...]:
        """The layers in the order in which they run."""
        count = len(self.layers)
        return (tuple(range(self.loop_start)) + tuple(range(self.loop_start, self.loop_stop)) * self.loop_times
                + tuple(range(self.loop_stop, count)))

    @classmethod
    def from_json(cls, raw: dict) -> "FasesunConfig":
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
            layers.append(LayerConfig(_mixer(entry["type"], _object(entry, "mixer", where), where + "mixer."),
                                      _mlp(entry.get("mlp"), where + "mlp")))
        loop = raw.get("loop")
        start, stop, times = 0, 0, 1
        if loop is not None:
            start, stop = _integer(loop, "start", "loop.", 0), _integer(loop, "stop", "loop.", 0)
            times = _integer(loop, "times", "loop.", 1)
            if not start <= stop <= len(layers):
                raise InvalidConfig(f"config.json: loop must satisfy 0 <= start <= stop <= {len(layers)}")
        return cls(vocab=_integer(raw, "vocab", ""), width=_integer(raw, "width", ""), eps=_number(_object(raw, "norm", ""), "eps", "norm."),
                   layers=tuple(layers), loop_start=start, loop_stop=stop, loop_times=times, declared_dtype=metadata.declared_dtype)
