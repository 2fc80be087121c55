"""Typed configuration of Pegurax, read from its own config.json keys.

A Pegurax folder names itself with `"architecture": "Pegurax"`.  `layers` lists the layers; each entry has a `type` (which mixer:
`parallel`, a softmax attention and a gated delta rule side by side; or `mamba1`, a selective scan), the mixer's sizes and constants
under `mixer` and its feed-forward under `mlp` (null: none; `kind` `dense` or `moe`).  `embedding.scale`, `norm.eps`, `vocab` and
`width` are model-wide.  Every size and constant that can differ between models is read here and nowhere else.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .bisudra import DenseConfig, MoEConfig, _mlp
from .errors import InvalidConfig
from .fasesun import _integer, _number, _object
from .metadata import metadata_from_json

ARCHITECTURE = "Pegurax"
MODEL_TYPE = "pegurax"
MIXER_TYPES = ("parallel", "mamba1")


@dataclass(frozen=True)
class RotationScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class SoftmaxSideConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotationScaling]


@dataclass(frozen=True)
class DeltaSideConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int


@dataclass(frozen=True)
class ParallelConfig:
    left: SoftmaxSideConfig
    right: DeltaSideConfig
    left_scale: float
    right_scale: float
    type: str = "parallel"


@dataclass(frozen=True)
class MambaConfig:
    inner: int
    states: int
    dt_rank: int
    taps: int
    type: str = "mamba1"


@dataclass(frozen=True)
class LayerConfig:
    mixer: object
    mlp: Optional[object]


def _heads(raw: dict, where: str):
    heads, kv_heads, dim, vdim = (_integer(raw, key, where) for key in ("heads", "kv_heads", "dim", "vdim"))
    if heads % kv_heads:
        raise InvalidConfig(f"config.json: {where}heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    return heads, kv_heads, dim, vdim


def _softmax_side(raw: dict, where: str) -> SoftmaxSideConfig:
    heads, kv_heads, dim, vdim = _heads(raw, where)
    rot = _object(raw, "rot", where) if raw.get("rot") is not None else {"dims": 0}       # no entry: nothing is rotated
    rot_dims = _integer(rot, "dims", where + "rot.", 0)
    if rot_dims % 2 or rot_dims > dim:
        raise InvalidConfig(f"config.json: {where}rot.dims must be even and at most dim ({dim}), found {rot_dims}")
    scaling = None
    if rot.get("scaling") is not None:
        listed = _object(rot, "scaling", where + "rot.")
        scaling = RotationScaling(*(_number(listed, key, where + "rot.scaling.") for key in ("factor", "original", "fast", "slow")))
    chunk = _integer(_object(raw, "mask", where), "size", where + "mask.") if raw.get("mask") is not None else 0     # no entry: every earlier position is seen
    return SoftmaxSideConfig(heads, kv_heads, dim, vdim, _number(raw, "scale", where), chunk,
                             _number(rot, "base", where + "rot.") if rot_dims else 1.0, rot_dims, scaling)


def _delta_side(raw: dict, where: str) -> DeltaSideConfig:
    heads, kv_heads, dim, vdim = _heads(raw, where)
    return DeltaSideConfig(heads, kv_heads, dim, vdim, _integer(raw, "conv", where))


def _mixer(kind: str, raw: dict, where: str):
    if kind == "parallel":
        return ParallelConfig(_softmax_side(_object(raw, "left", where), where + "left."), _delta_side(_object(raw, "right", where), where + "right."),
                              _number(raw, "left_scale", where, positive=False), _number(raw, "right_scale", where, positive=False))
    return MambaConfig(_integer(raw, "inner", where), _integer(raw, "state", where), _integer(raw, "dt_rank", where), _integer(raw, "conv", where))


@dataclass(frozen=True)
class PeguraxConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[LayerConfig, ...]
    declared_dtype: Optional[str] = None

    architecture = ARCHITECTURE
    model_type = MODEL_TYPE

    @classmethod
    def from_json(cls, raw: dict) -> "PeguraxConfig":
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
            layers.append(LayerConfig(_mixer(entry["type"], _object(entry, "mixer", where), where + "mixer."), _mlp(entry.get("mlp"), where + "mlp")))
        return cls(vocab=_integer(raw, "vocab", ""), width=_integer(raw, "width", ""), eps=_number(_object(raw, "norm", ""), "eps", "norm."),
                   embedding_scale=_number(_object(raw, "embedding", ""), "scale", "embedding.", positive=False), layers=tuple(layers),
                   declared_dtype=metadata.declared_dtype)


__all__ = ["ARCHITECTURE", "MODEL_TYPE", "DenseConfig", "MoEConfig", "PeguraxConfig"]
