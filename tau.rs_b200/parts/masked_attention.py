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

Two cache layouts, chosen from the sizes alone.  Where keys and values are equally wide and that width is one the tensor-core
kernel serves (`HEADS_LAYOUT_DIMS`), keys and values lie in pages of ordinary heads (`CacheNeed("kv")`): runs of new tokens in
bfloat16 then go through `attention_prefill_tc` (tcgen05; the mask, the sink and the scale are its parameters), everything else
(single tokens, 32-bit runs) through this mixer's own kernel, which reads either layout.  For any other sizes one row per position
is cached, `[keys of all kv heads | values of all kv heads]` (`CacheNeed("rows")`), and the mixer's own kernel serves every step.
The kernel that normalises and rotates writes the cache.  A sequence gives back the pages that lie wholly before its window or its
current chunk.  Scores, weights and sums are 32-bit.  Tensor names under the prefix: `q`, `k`, `v`, `o`, `q.norm`, `k.norm`.
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
        self.spec, self.prefix, self.dtype, self.device, self.hidden = spec, prefix, dtype, device, spec.hidden
        self.q_width, self.k_width, self.v_width = spec.n_heads * spec.dim, spec.n_kv_heads * spec.dim, spec.n_kv_heads * spec.value_dim
        self.position = None if spec.position is None else build("position", spec.position, device=device)
        if spec.position is not None and spec.position.rotary_dim > spec.dim:
            raise ValueError("the rotation is wider than a head")
        self.q_norm = self.k_norm = None
        self.heads_layout = spec.dim == spec.value_dim and spec.dim in HEADS_LAYOUT_DIMS
        self._finish_init(joined)

    def input_pieces(self):
        prefix = self.prefix
        return [(f"{prefix}.q", self.q_width), (f"{prefix}.k", self.k_width), (f"{prefix}.v", self.v_width)]

    @property
    def inner_features(self) -> int:
        return self.spec.n_heads * self.spec.value_dim

    def own_tensor_specs(self):
        if self.spec.qk_norm is None:
            return {}
        return {f"{self.prefix}.q.norm": TensorSpec((self.q_width,), role="vector", init="ones"),
                f"{self.prefix}.k.norm": TensorSpec((self.k_width,), role="vector", init="ones")}

    def finalize_own(self, held):
        if self.position is not None:
            self.position.finalize_weights()
        if self.spec.qk_norm is not None:
            self.q_norm, self.k_norm = held[f"{self.prefix}.q.norm"], held[f"{self.prefix}.k.norm"]

    def cache_need(self):
        if self.heads_layout:
            return CacheNeed("kv", n_kv_heads=self.spec.n_kv_heads, head_dim=self.spec.dim, window=self.spec.window, chunk=self.spec.chunk)
        return CacheNeed("rows", row_width=self.k_width + self.v_width, window=self.spec.window, chunk=self.spec.chunk)

    def mix(self, projected, gates, step, cache, writes_cache: bool, out) -> None:
        spec = self.spec
        tokens = projected.shape[0]
        queries = torch.empty((tokens, spec.n_heads, spec.dim), dtype=projected.dtype, device=projected.device)
        pages = step.page_rows[cache.group]
        position = self.position
        keys, values = (cache.keys, cache.values) if self.heads_layout else (cache.rows, None)
        kernels.masked_prepare(projected, self.q_norm, self.k_norm, spec.eps, None if position is None else position.frequency,
                               0 if position is None else spec.position.rotary_dim, 1.0 if position is None else position.magnitude, queries, keys,
                               step.positions, step.token_seq, pages, spec.n_heads, spec.n_kv_heads, spec.dim, spec.value_dim, writes_cache, values)
        if (self.heads_layout and not step.all_single and projected.dtype == torch.bfloat16 and kernels.optimized_preferred()
                and keys.shape[0] * spec.n_kv_heads * kernels.PAGE_TOKENS <= 0x7FFFFFFF and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0):
            kernels.attention_prefill_tc(queries.view(tokens, -1), keys, values, out, step.cu_seqlens, step.seq_start, pages, spec.n_heads, spec.n_kv_heads,
                                         spec.dim, spec.softmax_scale, spec.window or 0, spec.chunk or 0, spec.sink, self.out_scale)
            return
        kernels.masked_attention(queries, keys, out, step, pages, spec.n_kv_heads, spec.value_dim, spec.softmax_scale, spec.window or 0,
                                 spec.chunk or 0, spec.sink, self.out_scale, values, staged=step.all_single)
