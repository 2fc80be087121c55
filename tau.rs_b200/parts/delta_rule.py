"""The gated delta rule: a matrix state per head that decays, is corrected towards the token's value along the token's key, and is
read with the token's query (`DeltaRuleSpec`).

Per token, with `h` the mixer's input:
    q = W_q h, k = W_k h (key heads x key_dim), v = W_v h (heads x value_dim); value head a reads key head a / (heads / key heads)
    each of q, k, v passes a causal convolution over time per channel (`<name>.conv` [channels, taps], the last column weighing the
    token itself, zeros before the sequence's start) and SiLU
    q and k become unit vectors per head, x / sqrt(sum(x^2) + 1e-6); q also times key_dim^-1/2
    beta = sigmoid(W_b h);   g = exp(-exp(A_log) * softplus(W_a h + dt_bias)), one of each per head
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees the token's own write)
    out = W_o (o / rms(o) per head * norm * silu(W_g h))

The state (32-bit, [heads, value_dim, key_dim], zero when a sequence starts) lives in the cache's state group, the convolutions'
last `taps - 1` inputs (32-bit) in a second one (`extra_cache_needs()["taps"]`).  The products run in the run's dtype except the
two gate projections, which leave theirs in 32-bit; everything behind the convolutions is 32-bit.  One kernel walks a run of new
tokens of any length, so prompts, portions and single tokens are the same code.  Tensor names under the prefix: `q`, `k`, `v`, `g`,
`o`, `b`, `a`, `q.conv`, `k.conv`, `v.conv`, `A_log`, `dt_bias`, `norm`.

Options of the spec: a decay per head and key channel (`decay == "channel"`: `a` and `dt_bias` are `heads x key_dim` wide and g acts
on the rows of S one by one); the decay's pre-activation and the output gate through a few numbers each (`decay_rank`, `gate_rank`:
`a2 (a1 h)` and `g2 (g1 h)` instead of `a h` and `g h`; the first products ride with q, k and v, the second are small products of
their own, the decay's leaving in 32-bit); a sigmoid instead of SiLU on the output gate (`gate_activation`).
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import CacheNeed
from .registry import register_mixer
from .side_by_side import JoinableMixer


@register_mixer("gated_delta_rule")
class GatedDeltaRule(JoinableMixer):
    def __init__(self, spec, prefix: str, dtype, device, joined: bool = False):
        if spec.n_heads % spec.n_key_heads:
            raise ValueError("the key heads must divide the heads")
        if not 1 <= spec.key_dim <= kernels.DELTA_MAX_KEY_DIM:
            raise ValueError(f"key_dim must lie between 1 and {kernels.DELTA_MAX_KEY_DIM}")
        if spec.taps < 1:
            raise ValueError("a convolution has at least one tap")
        if spec.decay not in ("head", "channel"):
            raise ValueError(f"the decay is per 'head' or per 'channel', not {spec.decay!r}")
        if spec.gate_activation not in ("silu", "sigmoid"):
            raise ValueError(f"the output gate passes 'silu' or 'sigmoid', not {spec.gate_activation!r}")
        self.spec, self.prefix, self.dtype, self.device, self.hidden = spec, prefix, dtype, device, spec.hidden
        self.k_width, self.v_width = spec.n_key_heads * spec.key_dim, spec.n_heads * spec.value_dim
        self.conv_width = 2 * self.k_width + self.v_width
        self.decay_width = spec.n_heads * (spec.key_dim if spec.decay == "channel" else 1)
        self.taps_weight = self.a_log = self.dt_bias = self.norm_weight = None
        from .linear import StackedLinear

        names = dict(weight_suffix="", bias_suffix=".b")
        self.decay_up = StackedLinear([(f"{prefix}.a2", self.decay_width)], spec.decay_rank, False, dtype, device, **names) if spec.decay_rank else None
        self.gate_up = StackedLinear([(f"{prefix}.g2", self.v_width)], spec.gate_rank, False, dtype, device, **names) if spec.gate_rank else None
        self._low_rank = tuple(part for part in (self.decay_up, self.gate_up) if part is not None)
        self._finish_init(joined)

    # Run-dtype pieces: q, k, v, then the output gate (or its low-rank step), then the decay's low-rank step.  32-bit pieces: beta,
    # then the decay's pre-activation where it is a product of the input itself.
    def input_pieces(self):
        prefix, spec = self.prefix, self.spec
        pieces = [(f"{prefix}.q", self.k_width), (f"{prefix}.k", self.k_width), (f"{prefix}.v", self.v_width)]
        pieces.append((f"{prefix}.g1", spec.gate_rank) if spec.gate_rank else (f"{prefix}.g", self.v_width))
        if spec.decay_rank:
            pieces.append((f"{prefix}.a1", spec.decay_rank))
        return pieces

    def gate_pieces(self):
        pieces = [(f"{self.prefix}.b", self.spec.n_heads)]
        if not self.spec.decay_rank:
            pieces.append((f"{self.prefix}.a", self.decay_width))
        return pieces

    def tensor_specs(self):
        specs = super().tensor_specs()
        for part in self._low_rank:
            specs.update(part.tensor_specs())
        return specs

    def assign(self, name, tensor):
        for part in self._low_rank:
            if name in part.tensor_specs():
                return part.assign(name, tensor)
        return super().assign(name, tensor)

    def finalize_weights(self):
        for part in self._low_rank:
            part.finalize_weights()
        super().finalize_weights()

    @property
    def inner_features(self) -> int:
        return self.v_width

    def own_tensor_specs(self):
        prefix, spec = self.prefix, self.spec
        return {
            f"{prefix}.q.conv": TensorSpec((self.k_width, spec.taps), role="vector", std=0.3),
            f"{prefix}.k.conv": TensorSpec((self.k_width, spec.taps), role="vector", std=0.3),
            f"{prefix}.v.conv": TensorSpec((self.v_width, spec.taps), role="vector", std=0.3),
            f"{prefix}.A_log": TensorSpec((spec.n_heads,), role="vector", std=0.5),
            f"{prefix}.dt_bias": TensorSpec((self.decay_width,), role="vector", std=0.5),
            f"{prefix}.norm": TensorSpec((spec.value_dim,), role="vector", init="ones"),
        }

    def finalize_own(self, held):
        prefix, spec = self.prefix, self.spec
        # Stored [channels, taps]; the kernel reads tap by tap, the channels of q, k and v side by side.
        self.taps_weight = torch.cat([held[f"{prefix}.{name}.conv"] for name in ("q", "k", "v")], dim=0).t().contiguous()
        self.a_log, self.dt_bias = held[f"{prefix}.A_log"], held[f"{prefix}.dt_bias"]
        # One weight for all heads, and whatever multiplies the mixer's features (a neighbour's scale) with it.
        self.norm_weight = (held[f"{prefix}.norm"].repeat(spec.n_heads) * self.out_scale).contiguous()

    def cache_need(self):
        spec = self.spec
        return CacheNeed("state", state_shape=(spec.n_heads * spec.value_dim * spec.key_dim,), state_dtype=torch.float32)

    def extra_cache_needs(self):
        if self.spec.taps > 1:
            return {"taps": CacheNeed("state", state_shape=(self.spec.taps - 1, self.conv_width), state_dtype=torch.float32)}
        return {}

    def mix(self, projected, gates, step, cache, writes_cache: bool, out) -> None:
        spec = self.spec
        tokens, device = projected.shape[0], projected.device
        rows = torch.empty((tokens, self.conv_width), dtype=torch.float32, device=device)
        tail = cache.extra["taps"].state if spec.taps > 1 else None
        kernels.short_conv(projected[:, : self.conv_width], self.taps_weight, None, tail, step, rows, silu=True, update=writes_cache)
        gate_width = spec.gate_rank or self.v_width
        gate = projected[:, self.conv_width : self.conv_width + gate_width]
        if self.gate_up is not None:
            gate = self.gate_up.forward(gate)
        channel = None
        if spec.decay_rank:      # the decay's pre-activation through a few numbers; the second product leaves in 32-bit
            steps = self.decay_up.forward(projected[:, self.conv_width + gate_width : self.conv_width + gate_width + spec.decay_rank], out_dtype=torch.float32)
            if spec.decay == "channel":
                channel = steps
            else:
                gates = torch.cat([gates, steps], dim=1)
        elif spec.decay == "channel":
            channel = gates[:, spec.n_heads :].contiguous()
        decays = torch.empty((tokens, spec.n_heads, 2), dtype=torch.float32, device=device)
        key_query = torch.empty((tokens, spec.n_key_heads), dtype=torch.float32, device=device)
        kernels.delta_prepare(rows, 0, self.k_width, gates, self.a_log, self.dt_bias, decays, key_query, spec.n_heads, spec.n_key_heads, spec.key_dim, channel)
        read = torch.empty((tokens, self.v_width), dtype=torch.float32, device=device)
        kernels.delta_rule(rows, 0, self.k_width, 2 * self.k_width, decays, key_query, cache.state, step.cu_seqlens, step.seq_slot, read,
                           spec.n_heads, spec.n_key_heads, spec.key_dim, spec.value_dim, channel)
        kernels.gated_group_norm(read, self.norm_weight, gate, out, spec.n_heads, spec.eps, True, silu_gate=spec.gate_activation == "silu")
