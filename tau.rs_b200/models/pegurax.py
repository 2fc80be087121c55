"""Pegurax as a list of blocks: the only place that knows this architecture.

Every layer has a norm before and a norm behind each of its two sublayers and a layer scale on what they return
(`parts.block.SandwichBlock`), on a 32-bit residual stream that the embedding enters multiplied by a constant.  The mixer is either
two mixers side by side that read the same input (`parts.side_by_side.SideBySide`): a grouped-query softmax attention that sees
only its own chunk of positions, with a norm over the whole query and key projections, a scaled rotation and one added to the
softmax's denominator (`parts.masked_attention`), and a gated delta rule behind short convolutions (`parts.delta_rule`); or a
selective scan (`parts.selective_scan`).  The feed-forward is a gated one with ReLU, or routed experts (SiLU) whose sigmoid scores
weigh the chosen experts' inputs, or absent.  The norms are layer norms without bias.  Tensor names: `embed`, `l<i>.*`,
`final.norm`; the head is the embedding table (without the embedding's constant).
"""
from __future__ import annotations

from ..config.pegurax import ARCHITECTURE, MODEL_TYPE, PeguraxConfig
from ..config.registry import register_architecture
from ..config.specs import (DeltaRuleSpec, MaskedAttentionSpec, ModelSpec, NormSpec, RoutedExpertsSpec, SandwichBlockSpec, ScaledRotationSpec,
                            ScheduleEntry, SelectiveScanSpec, SideBySideSpec, SwiGLUSpec)

# The design numbers no positions and keeps no table over them; the limit is that of a 32-bit position.
MAX_POSITIONS = (1 << 31) - 1


def _mixer_spec(mixer, width: int, eps: float):
    if mixer.type == "mamba1":
        return SelectiveScanSpec(hidden=width, inner=mixer.inner, states=mixer.states, dt_rank=mixer.dt_rank, taps=mixer.taps)
    left, right = mixer.left, mixer.right
    position = None
    if left.rot_dims:
        scaling = left.rot_scaling
        position = ScaledRotationSpec(rotary_dim=left.rot_dims, theta=left.rot_base, factor=None if scaling is None else scaling.factor,
                                      original=0.0 if scaling is None else scaling.original, fast=0.0 if scaling is None else scaling.fast,
                                      slow=0.0 if scaling is None else scaling.slow)
    softmax = MaskedAttentionSpec(hidden=width, n_heads=left.heads, n_kv_heads=left.kv_heads, dim=left.dim, value_dim=left.vdim, softmax_scale=left.scale,
                                  eps=eps, qk_norm="projection", position=position, chunk=left.chunk or None, sink=True)
    delta = DeltaRuleSpec(hidden=width, n_heads=right.heads, n_key_heads=right.kv_heads, key_dim=right.dim, value_dim=right.vdim, taps=right.taps, eps=eps)
    return SideBySideSpec(left=softmax, right=delta, left_scale=mixer.left_scale, right_scale=mixer.right_scale)


def _feed_forward_spec(mlp, width: int):
    if mlp is None:
        return None
    if mlp.kind == "dense":
        return SwiGLUSpec(hidden=width, intermediate=mlp.ff, gate_name="gate", up_name="up", down_name="down", weight_suffix="", activation="relu")
    return RoutedExpertsSpec(hidden=width, intermediate=mlp.expert_ff, experts=mlp.experts, top=mlp.top, score="sigmoid", correction=False,
                             renormalize=False, shared=None, shared_gate=False, weigh="input")


def build_pegurax_spec(config: PeguraxConfig) -> ModelSpec:
    norm = NormSpec(width=config.width, eps=config.eps, kind="layer_norm", bias=False)
    blocks = tuple(
        SandwichBlockSpec(prefix=f"l{index}", mixer=_mixer_spec(layer.mixer, config.width, config.eps), feed_forward=_feed_forward_spec(layer.mlp, config.width),
                          mixer_norm=norm, mixer_post_norm=norm, feed_forward_norm=norm if layer.mlp is not None else None,
                          feed_forward_post_norm=norm if layer.mlp is not None else None, layer_scale=True)
        for index, layer in enumerate(config.layers)
    )
    # Layers whose mixers keep the same thing share a cache group, each with a cache layer of its own there; so does everything
    # that a mixer keeps beside its own cache (the other side's state, the convolutions' tails), role by role.
    schedule, counters, names = [], {}, {}

    def place(need_key, label):
        group = names.setdefault(need_key, f"{label}.{len(names)}")
        layer = counters.get(group, 0)
        counters[group] = layer + 1
        return group, layer

    for index, block in enumerate(blocks):
        mixer = block.mixer
        if mixer.kind == "side_by_side":
            group, layer = place(("keys", mixer.left), "keys")
            extra = [("right", *place(("delta", mixer.right.n_heads, mixer.right.key_dim, mixer.right.value_dim), "delta"))]
            if mixer.right.taps > 1:
                width = 2 * mixer.right.n_key_heads * mixer.right.key_dim + mixer.right.n_heads * mixer.right.value_dim
                extra.append(("right.taps", *place(("taps", mixer.right.taps, width), "taps")))
        else:
            group, layer = place(("scan", mixer.inner, mixer.states), "scan")
            extra = [("taps", *place(("taps", mixer.taps, mixer.inner), "taps"))] if mixer.taps > 1 else []
        schedule.append(ScheduleEntry(layer=index, cache_group=group, cache_layer=layer, writes_cache=True, extra_cache=tuple(extra)))
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=config.vocab, hidden=config.width, max_positions=MAX_POSITIONS, embedding_name="embed",
        blocks=blocks, schedule=tuple(schedule), final_norm=norm, final_norm_name="final.norm", head_name="head", tie_head=True,
        declared_dtype=config.declared_dtype, residual_dtype="float32", embedding_scale=config.embedding_scale,
    )


register_architecture(ARCHITECTURE, MODEL_TYPE, PeguraxConfig.from_json, build_pegurax_spec, storage_dtype="bfloat16")
