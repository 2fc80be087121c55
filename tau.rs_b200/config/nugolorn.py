"""Typed configuration of Nugolorn, read from its own config.json keys.

A Nugolorn folder names itself with `"architecture": "Nugolorn"`.  `layers` lists the layers; each entry has a `type` (which mixer:
`attention`, sigmoid-weighted attention behind short convolutions; `wkv`, a matrix memory with a decay per key channel; or
`parallel`, a softmax attention with a distance bias beside a gated delta rule), the mixer's sizes and constants under `mixer` and its
feed-forward under `mlp` (null: none; `kind` `dense` or `moe`, the latter with `router.identity` experts that return their input).
`norm.eps`, `norm.groups`, `residual_mult`, `logit_scale`, `vocab` and `width` are model-wide.  Every size and constant that can differ
between models is read here and nowhere else.  Three sizes are not in config.json but in the shapes of tensors, the numbers through
which the low-rank projections pass (`w1` of a `wkv` mixer, `a1` and `g1` of a delta rule): `sizes_from_tensors` writes them into the
configuration (`decay_rank`, `gate_rank`) before it is parsed; a configuration that carries them needs no folder.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

from .bisudra import DenseConfig
from .errors import InvalidConfig
from .fasesun import _integer, _number, _object
from .metadata import metadata_from_json

ARCHITECTURE = "Nugolorn"
MODEL_TYPE = "nugolorn"
MIXER_TYPES = ("attention", "wkv", "parallel")


@dataclass(frozen=True)
class SigmoidAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    taps: int
    rot_base: float
    rot_dims: int
    kv_from: Optional[int]
    type: str = "attention"


@dataclass(frozen=True)
class MemoryConfig:
    heads: int
    dim: int
    decay_rank: int
    type: str = "wkv"


@dataclass(frozen=True)
class DistanceAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temperature: Optional[Tuple[float, int]]


@dataclass(frozen=True)
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    decay_rank: int
    gate_rank: int


@dataclass(frozen=True)
class ParallelConfig:
    left: DistanceAttentionConfig
    right: ChannelDeltaConfig
    type: str = "parallel"


@dataclass(frozen=True)
class IdentityMoEConfig:
    experts: int
    identity: int
    top: int
    expert_ff: int
    kind: str = "moe"


@dataclass(frozen=True)
class LayerConfig:
    mixer: object
    mlp: Optional[object]


def _heads(raw: dict, where: str):
    heads, kv_heads, dim, vdim = (_integer(raw, key, where) for key in ("heads", "kv_heads", "dim", "vdim"))
    if heads % kv_heads:
        raise InvalidConfig(f"config.json: {where}heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    return heads, kv_heads, dim, vdim


def _attention(raw: dict, where: str, index: int) -> SigmoidAttentionConfig:
    heads, kv_heads, dim, vdim = _heads(raw, where)
    rot = _object(raw, "rot", where) if raw.get("rot") is not None else {"dims": 0}       # no entry: nothing is rotated
    rot_dims = _integer(rot, "dims", where + "rot.", 0)
    if rot_dims % 2 or rot_dims > dim:
        raise InvalidConfig(f"config.json: {where}rot.dims must be even and at most dim ({dim}), found {rot_dims}")
    kv_from = raw.get("kv_from")
    if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < index):
        raise InvalidConfig(f"config.json: {where}kv_from must name an earlier layer, found {kv_from!r}")
    return SigmoidAttentionConfig(heads, kv_heads, dim, vdim, _number(raw, "scale", where), _integer(raw, "conv", where) if raw.get("conv") is not None else 0,
                                  _number(rot, "base", where + "rot.") if rot_dims else 1.0, rot_dims, kv_from)


def _rank(raw: dict, key: str, where: str) -> int:
    if raw.get(key) is None:
        raise InvalidConfig(f"config.json: {where}{key!r} is neither given nor known from a tensor's shape (a folder's tensors give it)")
    return _integer(raw, key, where)


def _parallel(raw: dict, where: str) -> ParallelConfig:
    left, right = _object(raw, "left", where), _object(raw, "right", where)
    temperature = None
    if left.get("q_temp") is not None:
        listed = _object(left, "q_temp", where + "left.")
        temperature = (_number(listed, "coef", where + "left.q_temp.", positive=False), _integer(listed, "every", where + "left.q_temp."))
    softmax = DistanceAttentionConfig(*_heads(left, where + "left."), _number(left, "scale", where + "left."), temperature)
    delta = ChannelDeltaConfig(*_heads(right, where + "right."), _integer(right, "conv", where + "right."), _rank(right, "decay_rank", where + "right."),
                               _rank(right, "gate_rank", where + "right."))
    return ParallelConfig(softmax, delta)


def _mlp(raw, where: str):
    if raw is None:
        return None
    if not isinstance(raw, dict) or raw.get("kind") not in ("dense", "moe"):
        raise InvalidConfig(f"config.json: {where} must be null or an object of kind 'dense' or 'moe'")
    if raw["kind"] == "dense":
        return DenseConfig(_integer(raw, "ff", where + "."))
    router = _object(raw, "router", where + ".")
    experts, top = _integer(router, "experts", where + ".router."), _integer(router, "top", where + ".router.")
    identity = _integer(router, "identity", where + ".router.", 0) if router.get("identity") is not None else 0
    if top > experts + identity:
        raise InvalidConfig(f"config.json: {where}.router.top ({top}) exceeds the router's outputs ({experts + identity})")
    return IdentityMoEConfig(experts, identity, top, _integer(_object(raw, "expert", where + "."), "ff", where + ".expert."))


def sizes_from_tensors(raw: dict, shapes: Dict[str, Tuple[int, ...]]) -> dict:
    """`raw` with the sizes that only tensors' shapes give written into its mixers, where config.json leaves them out."""
    raw = copy.deepcopy(raw)
    for index, entry in enumerate(raw.get("layers") or []):
        if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
            continue
        mixer, prefix = entry["mixer"], f"l{index}.mix"

        def first_extent(name):
            shape = shapes.get(name)
            return int(shape[0]) if shape else None

        if entry.get("type") == "wkv" and mixer.get("decay_rank") is None:
            mixer["decay_rank"] = first_extent(f"{prefix}.w1")
        if entry.get("type") == "parallel" and isinstance(mixer.get("right"), dict):
            right = mixer["right"]
            if right.get("decay_rank") is None:
                right["decay_rank"] = first_extent(f"{prefix}.right.a1")
            if right.get("gate_rank") is None:
                right["gate_rank"] = first_extent(f"{prefix}.right.g1")
    return raw


@dataclass(frozen=True)
class NugolornConfig:
    vocab: int
    width: int
    eps: float
    groups: int
    residual_mult: float
    logit_scale: float
    layers: Tuple[LayerConfig, ...]
    declared_dtype: Optional[str] = None

    architecture = ARCHITECTURE
    model_type = MODEL_TYPE

    @classmethod
    def from_json(cls, raw: dict) -> "NugolornConfig":
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
            raw_mixer = _object(entry, "mixer", where)
            if entry["type"] == "attention":
                mixer = _attention(raw_mixer, where + "mixer.", index)
                if mixer.kv_from is not None:
                    source = layers[mixer.kv_from].mixer
                    if (source.type != "attention" or source.kv_from is not None
                            or (source.kv_heads, source.dim, source.vdim, source.rot_dims, source.rot_base) != (mixer.kv_heads, mixer.dim, mixer.vdim, mixer.rot_dims, mixer.rot_base)):
                        raise InvalidConfig(f"config.json: {where}mixer.kv_from must name an attention layer with keys and values of its own and of the same sizes")
            elif entry["type"] == "wkv":
                mixer = MemoryConfig(_integer(raw_mixer, "heads", where + "mixer."), _integer(raw_mixer, "dim", where + "mixer."), _rank(raw_mixer, "decay_rank", where + "mixer."))
            else:
                mixer = _parallel(raw_mixer, where + "mixer.")
            layers.append(LayerConfig(mixer, _mlp(entry.get("mlp"), where + "mlp")))
        norm = _object(raw, "norm", "")
        width = _integer(raw, "width", "")
        groups = _integer(norm, "groups", "norm.") if norm.get("groups") is not None else 1
        if width % groups:
            raise InvalidConfig(f"config.json: norm.groups ({groups}) must divide width ({width})")
        return cls(vocab=_integer(raw, "vocab", ""), width=width, eps=_number(norm, "eps", "norm."), groups=groups,
                   residual_mult=_number(raw, "residual_mult", "", positive=False) if raw.get("residual_mult") is not None else 1.0,
                   logit_scale=_number(raw, "logit_scale", "", positive=False) if raw.get("logit_scale") is not None else 1.0,
                   layers=tuple(layers), declared_dtype=metadata.declared_dtype)


__all__ = ["ARCHITECTURE", "MODEL_TYPE", "NugolornConfig", "sizes_from_tensors"]
