"""RMSNorm: `x * rsqrt(mean(x^2) + eps) * w`, statistic in 32-bit, one rounding; with `groups` > 1 each of that many equal
consecutive pieces of the row is divided by its own root mean square.

crates/models/src/components/rms_norm.rs:205-210 and :147-150; the in-tree norm scales
by `1 + w`, this part by `w`.  The fused form first rounds `residual + branch` to the
storage dtype and normalises that (rms_norm.rs:39-74;
crates/cuda-kernels/src/kernels/centered_rms_norm.cu:267-308).
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import Norm
from .registry import register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    def __init__(self, spec, name: str, dtype, device):
        self.spec, self.name = spec, name
        self.dtype = dtype      # of the output; the input may be a residual stream kept in 32-bit
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.spec.width,), role="vector", init="ones")}

    def assign(self, name, tensor):
        if name != self.name:
            raise KeyError(name)
        self.weight = tensor

    def _options(self, branch) -> dict:
        """What only some models ask of the kernel: pieces of the row normalised one by one, a factor on what joins the stream."""
        groups, scale = getattr(self.spec, "groups", 1), getattr(branch, "scale", 1.0)
        options = {} if groups == 1 else {"groups": groups}
        if scale != 1.0:
            options["branch_scale"] = scale
        return options

    def forward(self, values, rows=None, branch=None):
        count = values.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((count, self.spec.width), dtype=self.dtype or values.dtype, device=values.device)
        kernels.rms_norm(values, self.weight, self.spec.eps, out, rows, branch, **self._options(branch))
        return out

    def add_forward(self, branch, residual):
        out = torch.empty(residual.shape, dtype=self.dtype or residual.dtype, device=residual.device)
        kernels.add_rms_norm(branch, residual, self.weight, self.spec.eps, out, **self._options(branch))
        return out


@register_norm("layer_norm")
class LayerNorm(Norm):
    """`(x - mean) / sqrt(variance + eps) * w + b`, the variance being the mean of the squared deviations; statistics in 32-bit,
    one rounding.  The bias is the tensor `<name><spec.bias_suffix>`.  The input may be a residual stream kept in 32-bit."""

    def __init__(self, spec, name: str, dtype, device):
        self.spec, self.name, self.bias_name = spec, name, name + spec.bias_suffix
        self.dtype = dtype
        self.weight = self.bias = None

    def tensor_specs(self):
        width = self.spec.width
        specs = {self.name: TensorSpec((width,), role="vector", init="ones")}
        if getattr(self.spec, "bias", True):
            specs[self.bias_name] = TensorSpec((width,), role="vector")
        return specs

    def assign(self, name, tensor):
        if name == self.name:
            self.weight = tensor
        elif name == self.bias_name and getattr(self.spec, "bias", True):
            self.bias = tensor
        else:
            raise KeyError(name)

    def forward(self, values, rows=None, branch=None):
        if branch is not None:
            raise ValueError("a layer norm of this kind reads finished rows; a pending branch must be added first")
        count = values.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((count, self.spec.width), dtype=self.dtype or values.dtype, device=values.device)
        kernels.norm_rows(values, rows, self.weight, self.bias, self.spec.eps, True, out)
        return out
