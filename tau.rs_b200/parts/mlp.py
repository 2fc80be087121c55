"""Gated feed-forward: `down(act(gate(x)) * up(x))`, no biases; `act` is SiLU (SwiGLU) or, by the spec's `activation`, ReLU.

crates/models/src/components/mlp.rs:99-122,177-191; gate and up are one stacked product
followed by one fused activation kernel (crates/models/src/components/mlp/
projection.rs:123-143; crates/cuda-kernels/src/kernels/silu_and_mul.cu:51-76:
`out[r, c] = silu(in[r, c]) * in[r, I + c]`, in 32-bit with one rounding).
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from .base import FeedForward
from .linear import StackedLinear
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, spec, prefix: str, dtype, device):
        self.spec = spec
        self.activation = getattr(spec, "activation", "silu")
        if self.activation not in ("silu", "relu"):
            raise ValueError(f"unknown activation {self.activation!r}")
        # Where the gated product exists (bfloat16, aligned sizes; its epilogue is SiLU) gate and up rows are interleaved for it and
        # the activation is its epilogue; otherwise the two are stacked and the activation is a kernel of its own.
        self.fused = self.activation == "silu" and kernels.gated_fits(spec.hidden, spec.intermediate, dtype)
        gate, up, down = (getattr(spec, key, default) for key, default in (("gate_name", "gate_proj"), ("up_name", "up_proj"), ("down_name", "down_proj")))
        suffix = getattr(spec, "weight_suffix", ".weight")
        self.gate_up = StackedLinear(
            [(f"{prefix}.{gate}", spec.intermediate), (f"{prefix}.{up}", spec.intermediate)],
            spec.hidden, False, dtype, device, interleave=kernels.GATE_GROUP if self.fused else 0, weight_suffix=suffix,
        )
        self.down = StackedLinear([(f"{prefix}.{down}", spec.hidden)], spec.intermediate, False, dtype, device, weight_suffix=suffix)

    def tensor_specs(self):
        return {**self.gate_up.tensor_specs(), **self.down.tensor_specs()}

    def assign(self, name, tensor):
        part = self.gate_up if name in self.gate_up.tensor_specs() else self.down
        part.assign(name, tensor)

    def finalize_weights(self):
        self.gate_up.finalize_weights()
        self.down.finalize_weights()

    def forward(self, hidden, step):
        if self.fused:
            return self.down.forward(self.gate_up.forward_gated(hidden))
        stacked = self.gate_up.forward(hidden)
        activated = torch.empty((hidden.shape[0], self.spec.intermediate), dtype=hidden.dtype, device=hidden.device)
        kernels.silu_mul(stacked, activated, relu=self.activation == "relu")
        return self.down.forward(activated)


@register_feed_forward("dense_mlp")
class DenseFeedForward(FeedForward):
    """`down(act(up(x) + b_up)) + b_down`; the biases ride with the products, the activation is one kernel; the result is 32-bit."""

    def __init__(self, spec, prefix: str, dtype, device):
        if spec.activation != "relu_squared":
            raise ValueError(f"unknown activation {spec.activation!r}")
        self.spec = spec
        names = dict(weight_suffix=spec.weight_suffix, bias_suffix=spec.bias_suffix)
        self.up = StackedLinear([(f"{prefix}.{spec.up_name}", spec.intermediate)], spec.hidden, spec.bias, dtype, device, **names)
        self.down = StackedLinear([(f"{prefix}.{spec.down_name}", spec.hidden)], spec.intermediate, spec.bias, dtype, device, **names)

    def tensor_specs(self):
        return {**self.up.tensor_specs(), **self.down.tensor_specs()}

    def assign(self, name, tensor):
        part = self.up if name in self.up.tensor_specs() else self.down
        part.assign(name, tensor)

    def finalize_weights(self):
        self.up.finalize_weights()
        self.down.finalize_weights()

    def forward(self, hidden, step):
        inner = self.up.forward(hidden)
        kernels.relu_squared(inner, inner)
        return self.down.forward(inner, out_dtype=torch.float32)
