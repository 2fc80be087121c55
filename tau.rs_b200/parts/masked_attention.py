"""Grouped-query softmax attention with the mask, the denominator and the head sizes as parameters (`MaskedAttentionSpec`).

Per token, with `h` the mixer's input:
    q = W_q h (heads x dim), k = W_k h (kv_heads x dim), v = W_v h (kv_heads x value_dim); no biases
    `qk_norm == "projection"`: q, and k, are divided by the root mean square over their WHOLE projection (all heads at once) and
    multiplied by a weight of that size (`q.norm`, `k.norm`), before the rotation
    rotation of the first `rotary_dim` elements of every head of q and k (`position`, a `ScaledRotationSpec`)
    score(i, j) = (q_i . k_j) * softmax_scale for the keys j <= i that the mask lets through: the last `window` positions, or the
    positions of i's own chunk of `chunk` positions (chunks counted from position 0 of the sequence), or all
    softmax, with one added to the denominator if `sink`
    out = W_o (concatenated heads)

Options of the spec, each alone or together: biases on q, k and v (`bias`); a causal convolution of `taps` taps over time on every
channel of q, k and v directly behind the projection, before the rotation, whose last `taps - 1` inputs are state of the sequence
(`extra_cache_needs()["taps"]`); a query temperature that grows with the logarithm of the position (`temperature`); a bias on the
score that grows with the logarithm of the distance, `- r1 ln(1 + r2 (i - j))` per head (`distance_bias`); sigmoid weights instead of
a softmax, `sigmoid(score + pb[head])`, not normalised (`weights == "sigmoid"`); a sigmoid gate on the result from one more
projection of the input, one number per head or per element (`gate`); and no keys and values of its own (`own_keys=False`): the
layer's schedule entry then names the cache layer of another layer of the same sizes, whose cached keys (convolved and rotated)
and values it reads with its own queries.

Two cache layouts, chosen from the sizes alone.  Where keys and values are equally wide and that width is one the tensor-core
kernel serves (`HEADS_LAYOUT_DIMS`), keys and values lie in pages of ordinary heads (`CacheNeed("kv")`): runs of new tokens in
bfloat16 then go through `attention_prefill_tc` (tcgen05; the mask, the sink and the scale are its parameters), everything else
(single tokens, 32-bit runs) through this mixer's own kernel, which reads either layout.  For any other sizes one row per position
is cached, `[keys of all kv heads | values of all kv heads]` (`CacheNeed("rows")`), and the mixer's own kernel serves every step.
The kernel that normalises and rotates writes the cache.  A sequence gives back the pages that lie wholly before its window or its
current chunk.  Scores, weights and sums are 32-bit.  Tensor names under the prefix: `q`, `k`, `v`, `o`, `q.norm`, `k.norm`, `q.b`,
`k.b`, `v.b`, `q.conv`, `k.conv`, `v.conv`, `r1`, `r2`, `pb`, `g`.
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import CacheNeed
from .registry import build, register_mixer
from .side_by_side import JoinableMixer


HEADS_LAYOUT_DIMS = (64, 128)


@register_mixer("masked_attention")
class MaskedAttention(JoinableMixer):
    def __init__(self, spec, prefix: str, dtype, device, joined: bool = False):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError("the kv heads must divide the heads")
        if spec.qk_norm not in (None, "projection"):
            raise ValueError(f"unknown qk_norm {spec.qk_norm!r}")
        if spec.window and spec.chunk:
            raise ValueError("a window or a chunk, not both")
        if spec.value_dim > kernels.MASKED_MAX_VALUE_DIM:
            raise ValueError(f"value_dim may be at most {kernels.MASKED_MAX_VALUE_DIM}")
        if spec.weights not in ("softmax", "sigmoid"):
            raise ValueError(f"the weights are a 'softmax' or 'sigmoid', not {spec.weights!r}")
        if spec.weights == "sigmoid" and spec.sink:
            raise ValueError("sigmoid weights have no denominator for a sink to join")
        if spec.gate not in (None, "head", "element"):
            raise ValueError(f"the gate is per 'head' or per 'element', not {spec.gate!r}")
        if spec.taps < 0:
            raise ValueError("taps cannot be negative")
        if not spec.own_keys and spec.qk_norm is not None:
            raise ValueError("a layer that reads another's keys has no key norm of its own")
        self.spec, self.prefix, self.dtype, self.device, self.hidden = spec, prefix, dtype, device, spec.hidden
        self.q_width, self.k_width, self.v_width = spec.n_heads * spec.dim, spec.n_kv_heads * spec.dim, spec.n_kv_heads * spec.value_dim
        self.conv_width = self.q_width + (self.k_width + self.v_width if spec.own_keys else 0)      # what the products bring beside the gate
        self.gate_width = 0 if spec.gate is None else spec.n_heads * (1 if spec.gate == "head" else spec.value_dim)
        self.taps_weight = self.distance = self.head_offset = None
        self.position = None if spec.position is None else build("position", spec.position, device=device)
        if spec.position is not None and spec.position.rotary_dim > spec.dim:
            raise ValueError("the rotation is wider than a head")
        self.q_norm = self.k_norm = None
        self.heads_layout = spec.dim == spec.value_dim and spec.dim in HEADS_LAYOUT_DIMS
        self._finish_init(joined)

    def _projections(self):
        return ("q", "k", "v") if self.spec.own_keys else ("q",)

    def input_pieces(self):
        prefix = self.prefix
        widths = {"q": self.q_width, "k": self.k_width, "v": self.v_width}
        pieces = [(f"{prefix}.{name}", widths[name]) for name in self._projections()]
        return pieces + ([(f"{prefix}.g", self.gate_width)] if self.gate_width else [])

    def biased_pieces(self):
        return [f"{self.prefix}.{name}" for name in self._projections()] if self.spec.bias else []

    @property
    def inner_features(self) -> int:
        return self.spec.n_heads * self.spec.value_dim

    def own_tensor_specs(self):
        spec, prefix, specs = self.spec, self.prefix, {}
        if spec.qk_norm is not None:
            specs[f"{prefix}.q.norm"] = TensorSpec((self.q_width,), role="vector", init="ones")
            specs[f"{prefix}.k.norm"] = TensorSpec((self.k_width,), role="vector", init="ones")
        if spec.taps:
            widths = {"q": self.q_width, "k": self.k_width, "v": self.v_width}
            for name in self._projections():
                specs[f"{prefix}.{name}.conv"] = TensorSpec((widths[name], spec.taps), role="vector", std=0.3)
        if spec.distance_bias:
            specs[f"{prefix}.r1"] = TensorSpec((spec.n_heads,), role="vector", std=0.3)
            specs[f"{prefix}.r2"] = TensorSpec((spec.n_heads,), role="vector", init="ones")
        if spec.weights == "sigmoid":
            specs[f"{prefix}.pb"] = TensorSpec((spec.n_heads,), role="vector", std=0.5)
        return specs

    def finalize_own(self, held):
        spec, prefix = self.spec, self.prefix
        if self.position is not None:
            self.position.finalize_weights()
        if spec.qk_norm is not None:
            self.q_norm, self.k_norm = held[f"{prefix}.q.norm"], held[f"{prefix}.k.norm"]
        if spec.taps:      # stored [channels, taps]; the kernel reads tap by tap, the channels of q, k and v side by side
            self.taps_weight = torch.cat([held[f"{prefix}.{name}.conv"] for name in self._projections()], dim=0).t().contiguous()
        if spec.distance_bias:
            self.distance = torch.stack([held[f"{prefix}.r1"], held[f"{prefix}.r2"]], dim=1).contiguous()
        if spec.weights == "sigmoid":
            self.head_offset = held[f"{prefix}.pb"]

    def _splits(self, step) -> int:
        """Ranges that a step of single tokens cuts every context into: as many as fill the machine with the staged kernel's blocks (six
        to an SM), each at least 64 positions of what a token reads (its window or chunk bounds that), 32 at most.  Any number computes
        the same sums, so a captured graph that serves other lengths than the one it was captured at stays right."""
        if not step.all_single:
            return 1
        reach = min(step.max_len, self.spec.window or self.spec.chunk or step.max_len)
        return max(1, min(6 * kernels.sm_count() // max(1, step.n_seqs * self.decode_blocks()), reach // 64, 32))

    def extra_cache_needs(self):
        if self.spec.taps > 1:
            return {"taps": CacheNeed("state", state_shape=(self.spec.taps - 1, self.conv_width), state_dtype=torch.float32)}
        return {}

    def cache_need(self):
        if self.heads_layout:
            return CacheNeed("kv", n_kv_heads=self.spec.n_kv_heads, head_dim=self.spec.dim, window=self.spec.window, chunk=self.spec.chunk)
        return CacheNeed("rows", row_width=self.k_width + self.v_width, window=self.spec.window, chunk=self.spec.chunk)

    def decode_blocks(self):
        """Blocks of the staged kernel per sequence and context split: one per key/value head and pass over its query heads."""
        group = self.spec.n_heads // self.spec.n_kv_heads
        return self.spec.n_kv_heads * -(-group // kernels.MASKED_STAGED_WARPS)

    def mix(self, projected, gates, step, cache, writes_cache: bool, out) -> None:
        spec = self.spec
        tokens = projected.shape[0]
        queries = torch.empty((tokens, spec.n_heads, spec.dim), dtype=projected.dtype, device=projected.device)
        pages = step.page_rows[cache.group]
        position = self.position
        keys, values = (cache.keys, cache.values) if self.heads_layout else (cache.rows, None)
        gate = projected[:, self.conv_width : self.conv_width + self.gate_width] if self.gate_width else None
        if spec.taps:      # the convolutions' tail is the layer's own even where the keys and values are another's
            convolved = torch.empty((tokens, self.conv_width), dtype=projected.dtype, device=projected.device)
            kernels.short_conv(projected[:, : self.conv_width], self.taps_weight, None, cache.extra["taps"].state if spec.taps > 1 else None, step, convolved,
                               silu=False, update=True)
            projected = convolved
        kernels.masked_prepare(projected, self.q_norm, self.k_norm, spec.eps, None if position is None else position.frequency,
                               0 if position is None else spec.position.rotary_dim, 1.0 if position is None else position.magnitude, queries, keys,
                               step.positions, step.token_seq, pages, spec.n_heads, spec.n_kv_heads, spec.dim, spec.value_dim, writes_cache and spec.own_keys, values,
                               temperature=spec.temperature)
        if (self.heads_layout and not step.all_single and projected.dtype == torch.bfloat16 and kernels.optimized_preferred()
                and keys.shape[0] * spec.n_kv_heads * kernels.PAGE_TOKENS <= 0x7FFFFFFF and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0):
            # Runs of new tokens on the tensor cores; a gate per head leaves with the rows, a gate per element is a pass of its own.
            kernels.attention_prefill_tc(queries.view(tokens, -1), keys, values, out, step.cu_seqlens, step.seq_start, pages, spec.n_heads, spec.n_kv_heads,
                                         spec.dim, spec.softmax_scale, spec.window or 0, spec.chunk or 0, spec.sink, self.out_scale, distance=self.distance,
                                         sigmoid_weights=spec.weights == "sigmoid", head_offset=self.head_offset, head_gate=gate if spec.gate == "head" else None)
            if spec.gate == "element":
                kernels.gated_rows(out, gate, out)
            return
        kernels.masked_attention(queries, keys, out, step, pages, spec.n_kv_heads, spec.value_dim, spec.softmax_scale, spec.window or 0,
                                 spec.chunk or 0, spec.sink, self.out_scale, values, staged=step.all_single, splits=self._splits(step), distance=self.distance,
                                 sigmoid_weights=spec.weights == "sigmoid", head_offset=self.head_offset, gate=gate, gate_per_head=spec.gate == "head")
