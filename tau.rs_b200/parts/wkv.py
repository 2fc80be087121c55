"""Time mixing with a matrix state per head, a decay per key channel and a bonus for the token itself (`ChannelDecayMemorySpec`).

Per token, with `h` the mixer's input and `h'` the input of the token before it in the sequence (zeros for the first token):
    mix_s = h + (h' - h) * mu_s                          one mix per projection, s in (r, k, v, g, w)
    r = W_r mix_r, k = W_k mix_k, v = W_v mix_v          heads x key_dim each
    gate = silu(W_g mix_g)
    w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))            per head and key channel, through `decay_rank` numbers
    o = (S + diag(u) k v^T)^T r                          per head; the bonus u weighs the token's own k v^T in its own read-out only
    S <- diag(w) S + k v^T
    out = W_o (o / rms(o) per head * norm * gate)

The state S (32-bit, [heads, key_dim, key_dim], zero when a sequence starts) lives in the cache's state group and the sequence's last
input `h` (kept in 32-bit) in a second one (`extra_cache_needs()["shift"]`).  The products run in the run's dtype; r, k, v and the
decay's pre-activation leave theirs in 32-bit, and the decay, the walk, the per-head norm and the gate are 32-bit.  One kernel walks a
run of new tokens of any length, so prompts, portions and single tokens are the same code.  Tensor names under the prefix: `mu.r`,
`mu.k`, `mu.v`, `mu.g`, `mu.w`, `r`, `k`, `v`, `g`, `w1`, `w2`, `w0`, `u`, `norm`, `o`.
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import CacheNeed, Mixer
from .linear import StackedLinear
from .registry import register_mixer

_MIXES = ("r", "k", "v", "g", "w")
_PLAIN = dict(weight_suffix="", bias_suffix=".b")


@register_mixer("channel_decay_memory")
class ChannelDecayMemory(Mixer):
    def __init__(self, spec, prefix: str, dtype, device):
        if not 1 <= spec.key_dim <= kernels.WKV_MAX_KEY_DIM:
            raise ValueError(f"key_dim must lie between 1 and {kernels.WKV_MAX_KEY_DIM}")
        if spec.decay_rank < 1:
            raise ValueError("the decay passes through at least one number")
        self.spec, self.prefix, self.dtype, self.device = spec, prefix, dtype, device
        self.inner = spec.n_heads * spec.key_dim
        hidden, inner = spec.hidden, self.inner
        self.products = {name: StackedLinear([(f"{prefix}.{name}", inner)], hidden, False, dtype, device, **_PLAIN) for name in ("r", "k", "v", "g")}
        self.decay_down = StackedLinear([(f"{prefix}.w1", spec.decay_rank)], hidden, False, dtype, device, **_PLAIN)
        self.decay_up = StackedLinear([(f"{prefix}.w2", inner)], spec.decay_rank, False, dtype, device, **_PLAIN)
        self.out = StackedLinear([(f"{prefix}.o", hidden)], inner, False, dtype, device, **_PLAIN)
        self._linears = (*self.products.values(), self.decay_down, self.decay_up, self.out)
        self._own = {f"{prefix}.mu.{name}": TensorSpec((hidden,), role="vector", std=0.3) for name in _MIXES}
        self._own[f"{prefix}.w0"] = TensorSpec((inner,), role="vector", std=0.5)
        self._own[f"{prefix}.u"] = TensorSpec((spec.n_heads, spec.key_dim), role="vector", std=0.3)
        self._own[f"{prefix}.norm"] = TensorSpec((inner,), role="vector", init="ones")
        self._held = {}
        self.mixes = self.decay_offset = self.bonus = self.norm_weight = None

    def tensor_specs(self):
        specs = dict(self._own)
        for part in self._linears:
            specs.update(part.tensor_specs())
        return specs

    def assign(self, name, tensor):
        if name in self._own:
            self._held[name] = tensor
            return
        for part in self._linears:
            if name in part.tensor_specs():
                return part.assign(name, tensor)
        raise KeyError(name)

    def finalize_weights(self):
        prefix, held = self.prefix, self._held
        for part in self._linears:
            part.finalize_weights()
        self.mixes = torch.stack([held.pop(f"{prefix}.mu.{name}") for name in _MIXES]).contiguous()
        self.decay_offset, self.bonus, self.norm_weight = held.pop(f"{prefix}.w0"), held.pop(f"{prefix}.u").contiguous(), held.pop(f"{prefix}.norm")

    def cache_need(self):
        spec = self.spec
        return CacheNeed("state", state_shape=(spec.n_heads * spec.key_dim * spec.key_dim,), state_dtype=torch.float32)

    def extra_cache_needs(self):
        return {"shift": CacheNeed("state", state_shape=(self.spec.hidden,), state_dtype=torch.float32)}

    def forward(self, hidden, step, cache, writes_cache: bool):
        spec = self.spec
        tokens, device = hidden.shape[0], hidden.device
        mixed = torch.empty((len(_MIXES), tokens, spec.hidden), dtype=hidden.dtype, device=device)
        kernels.token_shift(hidden, self.mixes, cache.extra["shift"].state, step, mixed, update=writes_cache)
        r, k, v = (self.products[name].forward(mixed[index], out_dtype=torch.float32) for index, name in enumerate(("r", "k", "v")))
        gate = self.products["g"].forward(mixed[3])
        low = self.decay_down.forward(mixed[4])
        kernels.tanh_(low)
        decay = self.decay_up.forward(low, out_dtype=torch.float32)
        kernels.channel_decay(decay, self.decay_offset)
        read = torch.empty((tokens, self.inner), dtype=torch.float32, device=device)
        kernels.wkv(r, k, v, decay, self.bonus, cache.state, step.cu_seqlens, step.seq_slot, read, spec.n_heads, spec.key_dim, spec.key_dim)
        features = torch.empty((tokens, self.inner), dtype=hidden.dtype, device=device)
        kernels.gated_group_norm(read, self.norm_weight, gate, features, spec.n_heads, spec.eps, True, silu_gate=True)
        return self.out.forward(features, out_dtype=torch.float32)
