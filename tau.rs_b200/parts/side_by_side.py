"""Mixers that can share their products with a neighbour, and the mixer that sets two of them side by side.

A `JoinableMixer` says which projections of its input it needs (`input_pieces`: in the run's dtype; `gate_pieces`: in 32-bit), how
wide the features are that its output projection reads (`inner_features`) and what that projection's tensor is called
(`output_name`); `mix()` turns the projections into those features, written into a column range that the caller provides.  Alone,
such a mixer stacks its own pieces into one product (two with gates) and applies its own output projection.  `SideBySide` holds two
of them that read the same input: all pieces of both become one stacked product (the 32-bit ones a second), each mixer writes its
features, already multiplied by its scale, beside the other's, and one product over `[left features | right features]` with the two
output weights set side by side along their input axis gives `left_scale * left + right_scale * right`.  Where the two results are
normalised before they are added (`join == "normed"`) each side has a product of its own and one kernel normalises, weighs and adds.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import CacheNeed, Mixer
from .linear import StackedLinear
from .registry import build, register_mixer

_PLAIN = dict(weight_suffix="", bias_suffix=".b")


class JoinableMixer(Mixer):
    """Subclasses set `spec`, `prefix`, `dtype`, `device`, `hidden`, then call `_finish_init(joined)`."""

    out_scale = 1.0     # multiplies the features that the output projection reads; set by whoever joins this mixer with another

    # ---- what a subclass states --------------------------------------------------
    def input_pieces(self) -> List[Tuple[str, int]]:
        raise NotImplementedError

    def gate_pieces(self) -> List[Tuple[str, int]]:
        return []

    def biased_pieces(self) -> List[str]:
        """The input pieces that have a bias tensor (`<piece>.b`)."""
        return []

    @property
    def inner_features(self) -> int:
        raise NotImplementedError

    @property
    def output_name(self) -> str:
        return f"{self.prefix}.o"

    def own_tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def finalize_own(self, held: Dict[str, torch.Tensor]) -> None:
        pass

    def mix(self, projected, gates, step, cache, writes_cache: bool, out) -> None:
        """`projected` [tokens, sum of input pieces] (run dtype), `gates` [tokens, sum of gate pieces] float32 or None; writes
        `out` [tokens, inner_features] (rows any distance apart)."""
        raise NotImplementedError

    # ---- shared machinery --------------------------------------------------------
    def _finish_init(self, joined: bool) -> None:
        self.joined = joined
        self._held: Dict[str, torch.Tensor] = {}
        self.inputs = self.gates = self.out = None
        if not joined:
            biased = self.biased_pieces()
            self.inputs = StackedLinear(self.input_pieces(), self.hidden, bool(biased), self.dtype, self.device, biased=biased or None, **_PLAIN)
            if self.gate_pieces():
                self.gates = StackedLinear(self.gate_pieces(), self.hidden, False, self.dtype, self.device, **_PLAIN)
            self.out = StackedLinear([(self.output_name, self.hidden)], self.inner_features, False, self.dtype, self.device, **_PLAIN)
        self._linears = tuple(part for part in (self.inputs, self.gates, self.out) if part is not None)

    def tensor_specs(self):
        specs = dict(self.own_tensor_specs())
        for part in self._linears:
            specs.update(part.tensor_specs())
        return specs

    def assign(self, name, tensor):
        if name in self.own_tensor_specs():
            self._held[name] = tensor
            return
        for part in self._linears:
            if name in part.tensor_specs():
                return part.assign(name, tensor)
        raise KeyError(name)

    def finalize_weights(self):
        for part in self._linears:
            part.finalize_weights()
        self.finalize_own(self._held)
        self._held = {}

    def forward(self, hidden, step, cache, writes_cache: bool):
        projected = self.inputs.forward(hidden)
        gates = None if self.gates is None else self.gates.forward(hidden, out_dtype=torch.float32)
        features = torch.empty((hidden.shape[0], self.inner_features), dtype=hidden.dtype, device=hidden.device)
        self.mix(projected, gates, step, cache, writes_cache, features)
        return self.out.forward(features, out_dtype=torch.float32)


class _RoleView:
    """What a joined mixer sees as its cache: one view, with the views of what it keeps beside it under `extra`."""

    def __init__(self, view, extra):
        self.__dict__.update(view.__dict__)
        self.extra = extra


@register_mixer("side_by_side")
class SideBySide(Mixer):
    def __init__(self, spec, prefix: str, dtype, device):
        self.spec, self.prefix, self.dtype, self.device = spec, prefix, dtype, device
        self.left = build("mixer", spec.left, prefix=f"{prefix}.{spec.left_name}", dtype=dtype, device=device, joined=True)
        self.right = build("mixer", spec.right, prefix=f"{prefix}.{spec.right_name}", dtype=dtype, device=device, joined=True)
        self.sides = (self.left, self.right)
        if getattr(spec, "join", "sum") == "sum":      # (joined behind norms, the scales multiply the normalised results instead)
            self.left.out_scale, self.right.out_scale = float(spec.left_scale), float(spec.right_scale)
        hidden = self.left.hidden
        if self.right.hidden != hidden:
            raise ValueError("the two mixers must read the same width")
        self.hidden = hidden
        biased = [name for side in self.sides for name in side.biased_pieces()]
        self.inputs = StackedLinear([piece for side in self.sides for piece in side.input_pieces()], hidden, bool(biased), dtype, device, biased=biased or None, **_PLAIN)
        gate_pieces = [piece for side in self.sides for piece in side.gate_pieces()]
        self.gates = StackedLinear(gate_pieces, hidden, False, dtype, device, **_PLAIN) if gate_pieces else None
        self._linears = tuple(part for part in (self.inputs, self.gates) if part is not None)
        if spec.join not in ("sum", "normed"):
            raise ValueError(f"the two results are joined as a 'sum' or 'normed', not {spec.join!r}")
        self._out_specs = {side.output_name: TensorSpec((hidden, side.inner_features), role="matrix") for side in self.sides}
        self._join_names = ()
        if spec.join == "normed":     # each side's result is normalised with a weight of its own before the two are added
            self._join_names = (f"{prefix}.{spec.left_name}.out", f"{prefix}.{spec.right_name}.out")
            self._out_specs.update({name: TensorSpec((hidden,), role="vector", init="ones") for name in self._join_names})
        self._held: Dict[str, torch.Tensor] = {}
        self.out_weight = self.out_weights = self.join_weights = None
        self.capturable = all(getattr(side, "capturable", True) for side in self.sides)

    # The left mixer's cache is the mixer's own; the right one's, and what either keeps beside, are kept under roles.
    def cache_need(self):
        return self.left.cache_need()

    def extra_cache_needs(self) -> Dict[str, CacheNeed]:
        needs = {f"left.{role}": need for role, need in self.left.extra_cache_needs().items()}
        if self.right.cache_need() is not None:
            needs["right"] = self.right.cache_need()
        needs.update({f"right.{role}": need for role, need in self.right.extra_cache_needs().items()})
        return needs

    def decode_blocks(self):
        return self.left.decode_blocks()

    def tensor_specs(self):
        specs = dict(self._out_specs)
        for part in (*self._linears, *self.sides):
            specs.update(part.tensor_specs())
        return specs

    def assign(self, name, tensor):
        if name in self._out_specs:
            self._held[name] = tensor
            return
        for part in (*self._linears, *self.sides):
            if name in part.tensor_specs():
                return part.assign(name, tensor)
        raise KeyError(name)

    def finalize_weights(self):
        for part in (*self._linears, *self.sides):
            part.finalize_weights()
        if self.spec.join == "normed":      # a product per side: the norms stand between the projections and the sum
            self.out_weights = tuple(self._held.pop(side.output_name) for side in self.sides)
            self.join_weights = tuple(self._held.pop(name) for name in self._join_names)
            return
        # [hidden, left features | right features]: one product over both mixers' features is the sum of their projections.
        self.out_weight = torch.cat([self._held.pop(side.output_name) for side in self.sides], dim=1).contiguous()

    def forward(self, hidden, step, cache, writes_cache: bool):
        tokens, device = hidden.shape[0], hidden.device
        projected = self.inputs.forward(hidden)
        gates = None if self.gates is None else self.gates.forward(hidden, out_dtype=torch.float32)
        normed = self.spec.join == "normed"
        if normed:      # a tensor of features per side, for a product per side
            targets = [torch.empty((tokens, side.inner_features), dtype=hidden.dtype, device=device) for side in self.sides]
        else:
            features = torch.empty((tokens, self.out_weight.shape[1]), dtype=hidden.dtype, device=device)
            left_features = self.left.inner_features
            targets = [features[:, :left_features], features[:, left_features:]]
        extra = getattr(cache, "extra", {}) if cache is not None else {}
        column = gate_column = 0
        for name, side, target in (("left", self.left, targets[0]), ("right", self.right, targets[1])):
            width = sum(size for _, size in side.input_pieces())
            gate_width = sum(size for _, size in side.gate_pieces())
            own = {role[len(name) + 1:]: view for role, view in extra.items() if role.startswith(name + ".")}
            view = cache if name == "left" else extra.get("right")
            side.mix(projected[:, column : column + width], None if not gate_width else gates[:, gate_column : gate_column + gate_width],
                     step, None if view is None else _RoleView(view, own), writes_cache, target)
            column, gate_column = column + width, gate_column + gate_width
        out = torch.empty((tokens, self.hidden), dtype=torch.float32, device=device)
        if normed:
            results = []
            for target, weight in zip(targets, self.out_weights):
                result = torch.empty((tokens, self.hidden), dtype=torch.float32, device=device)
                kernels.linear(target, weight, None, result)
                results.append(result)
            kernels.normed_pair_sum(results[0], results[1], self.join_weights[0], self.join_weights[1], self.spec.eps, float(self.spec.left_scale),
                                    float(self.spec.right_scale), out)
            return out
        kernels.linear(features, self.out_weight, None, out)
        return out
