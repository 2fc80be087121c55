"""A Mamba mixer: a selective scan over a widened copy of the input, gated by a second copy (`SelectiveScanSpec`).

Per token, with `h` the mixer's input:
    [x | z] = W_in h (inner each);   x passes a causal convolution over time per channel (`conv` [inner, taps] with bias `conv.b`,
    the last column weighing the token itself, zeros before the sequence's start) and SiLU
    [dt | B | C] = W_x x (dt_rank, states, states);   step = softplus(W_dt dt + b_dt), one per channel;   A = -exp(A_log)
    S[c, n] <- exp(step_c A[c, n]) S[c, n] + step_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c
    out = W_o (y * silu(z))

The state (32-bit, [inner, states], zero when a sequence starts) lives in the cache's state group, the convolution's last
`taps - 1` inputs (32-bit) in a second one (`extra_cache_needs()["taps"]`).  `W_x` is applied as two products so that B and C leave
theirs in 32-bit while `dt` feeds the next product in the run's dtype; the step sizes' pre-activations, the softplus, the
exponentials, the state and the read-out are 32-bit.  One kernel walks a run of new tokens of any length.  Tensor names under the
prefix: `in`, `conv`, `conv.b`, `x`, `dt`, `dt.b`, `A_log`, `D`, `o`.
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import CacheNeed
from .registry import register_mixer
from .side_by_side import JoinableMixer


@register_mixer("selective_scan")
class SelectiveScan(JoinableMixer):
    def __init__(self, spec, prefix: str, dtype, device, joined: bool = False):
        if not 1 <= spec.states <= kernels.SCAN_MAX_STATES:
            raise ValueError(f"states must lie between 1 and {kernels.SCAN_MAX_STATES}")
        if spec.taps < 1 or spec.dt_rank < 1:
            raise ValueError("a convolution has at least one tap, and the step sizes at least one input")
        self.spec, self.prefix, self.dtype, self.device, self.hidden = spec, prefix, dtype, device, spec.hidden
        self.taps_weight = self.taps_bias = self.low_step = self.low_bc = self.step_weight = self.step_bias = self.a_log = self.skip = None
        self._finish_init(joined)

    def input_pieces(self):
        return [(f"{self.prefix}.in", 2 * self.spec.inner)]

    @property
    def inner_features(self) -> int:
        return self.spec.inner

    def own_tensor_specs(self):
        prefix, spec = self.prefix, self.spec
        return {
            f"{prefix}.conv": TensorSpec((spec.inner, spec.taps), role="vector", std=0.3),
            f"{prefix}.conv.b": TensorSpec((spec.inner,), role="vector", std=0.1),
            f"{prefix}.x": TensorSpec((spec.dt_rank + 2 * spec.states, spec.inner), role="matrix"),
            f"{prefix}.dt": TensorSpec((spec.inner, spec.dt_rank), role="matrix", std=0.2),
            f"{prefix}.dt.b": TensorSpec((spec.inner,), role="vector", std=0.5),
            f"{prefix}.A_log": TensorSpec((spec.inner, spec.states), role="vector", std=0.5),
            f"{prefix}.D": TensorSpec((spec.inner,), role="vector", init="ones"),
        }

    def finalize_own(self, held):
        prefix, spec = self.prefix, self.spec
        self.taps_weight = held[f"{prefix}.conv"].t().contiguous()        # tap by tap, a tap's channels side by side
        self.taps_bias = held[f"{prefix}.conv.b"]
        low = held[f"{prefix}.x"]
        self.low_step, self.low_bc = low[: spec.dt_rank].contiguous(), low[spec.dt_rank :].contiguous()
        self.step_weight, self.step_bias = held[f"{prefix}.dt"], held[f"{prefix}.dt.b"]
        self.a_log, self.skip = held[f"{prefix}.A_log"], held[f"{prefix}.D"]

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.spec.inner * self.spec.states,), state_dtype=torch.float32)

    def extra_cache_needs(self):
        if self.spec.taps > 1:
            return {"taps": CacheNeed("state", state_shape=(self.spec.taps - 1, self.spec.inner), state_dtype=torch.float32)}
        return {}

    def mix(self, projected, gates, step, cache, writes_cache: bool, out) -> None:
        spec = self.spec
        if self.out_scale != 1.0 or not out.is_contiguous():
            raise ValueError("this mixer writes whole rows and takes no scale on its features: it stands alone in its layer")
        tokens, device, inner = projected.shape[0], projected.device, spec.inner
        x = torch.empty((tokens, inner), dtype=projected.dtype, device=device)
        tail = cache.extra["taps"].state if spec.taps > 1 else None
        kernels.short_conv(projected[:, :inner], self.taps_weight, self.taps_bias, tail, step, x, silu=True, update=writes_cache)
        low = torch.empty((tokens, spec.dt_rank), dtype=projected.dtype, device=device)
        kernels.linear(x, self.low_step, None, low)
        drive = torch.empty((tokens, 2 * spec.states), dtype=torch.float32, device=device)
        kernels.linear(x, self.low_bc, None, drive)
        pre = torch.empty((tokens, inner), dtype=torch.float32, device=device)
        kernels.linear(low, self.step_weight, self.step_bias, pre)
        kernels.selective_scan(x, projected[:, inner:], pre, drive, self.a_log, self.skip, cache.state, step.cu_seqlens, step.seq_slot, out)
