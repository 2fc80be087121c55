"""Nugolorn as a list of blocks: the only place that knows this architecture.

Every layer is a parallel block (`parts.block.ParallelBlock`): one RMS norm in groups, the mixer and the feed-forward both read its
output, and their sum joins the 32-bit residual stream multiplied by a constant.  The mixer is one of three: attention whose q, k and
v have biases and pass short causal convolutions before a rotation of halves, whose visible keys weigh sigmoid(score + a number per
head) without a softmax, and whose heads are gated by one sigmoid each (`parts.masked_attention` with those options; such a layer may
read the keys and values that an earlier one cached instead of having its own); a matrix memory with a decay per key channel and a
bonus for the token itself behind a token shift (`parts.wkv`); or two mixers side by side (`parts.side_by_side`, joined behind a norm
each): a softmax attention without rotation whose queries grow with the logarithm of the position and whose scores fall with the
logarithm of the distance, gated element by element, and a gated delta rule with a decay per key channel whose decay and output gate
pass through low-rank projections (`parts.delta_rule` with those options).  The feed-forward is a gated one (SiLU), or routed experts
with a softmax router, a correction on the choice, weights that are not renormalised and identity experts, or absent.  Tensor names:
`embed`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.nugolorn import ARCHITECTURE, MODEL_TYPE, NugolornConfig, sizes_from_tensors
from ..config.registry import register_architecture
from ..config.specs import (BlockSpec, ChannelDecayMemorySpec, DeltaRuleSpec, MaskedAttentionSpec, ModelSpec, NormSpec, RoutedExpertsSpec, ScaledRotationSpec,
                            ScheduleEntry, SideBySideSpec, SwiGLUSpec)

# The design keeps no table over positions; the limit is that of a 32-bit position.
MAX_POSITIONS = (1 << 31) - 1


def _mixer_spec(mixer, width: int, eps: float):
    if mixer.type == "attention":
        position = ScaledRotationSpec(rotary_dim=mixer.rot_dims, theta=mixer.rot_base) if mixer.rot_dims else None
        return MaskedAttentionSpec(hidden=width, n_heads=mixer.heads, n_kv_heads=mixer.kv_heads, dim=mixer.dim, value_dim=mixer.vdim, softmax_scale=mixer.scale,
                                   eps=eps, position=position, bias=True, taps=mixer.taps, weights="sigmoid", gate="head", own_keys=mixer.kv_from is None)
    if mixer.type == "wkv":
        return ChannelDecayMemorySpec(hidden=width, n_heads=mixer.heads, key_dim=mixer.dim, decay_rank=mixer.decay_rank, eps=eps)
    left, right = mixer.left, mixer.right
    softmax = MaskedAttentionSpec(hidden=width, n_heads=left.heads, n_kv_heads=left.kv_heads, dim=left.dim, value_dim=left.vdim, softmax_scale=left.scale,
                                  eps=eps, temperature=left.temperature, distance_bias=True, gate="element")
    delta = DeltaRuleSpec(hidden=width, n_heads=right.heads, n_key_heads=right.kv_heads, key_dim=right.dim, value_dim=right.vdim, taps=right.taps, eps=eps,
                          decay="channel", decay_rank=right.decay_rank, gate_rank=right.gate_rank, gate_activation="sigmoid")
    return SideBySideSpec(left=softmax, right=delta, left_scale=0.5, right_scale=0.5, join="normed", eps=eps)


def _feed_forward_spec(mlp, width: int):
    if mlp is None:
        return None
    if mlp.kind == "dense":
        return SwiGLUSpec(hidden=width, intermediate=mlp.ff, gate_name="gate", up_name="up", down_name="down", weight_suffix="")
    return RoutedExpertsSpec(hidden=width, intermediate=mlp.expert_ff, experts=mlp.experts, top=mlp.top, score="softmax", correction=True,
                             renormalize=False, shared=None, shared_gate=False, identity=mlp.identity)


def build_nugolorn_spec(config: NugolornConfig) -> ModelSpec:
    norm = NormSpec(width=config.width, eps=config.eps, groups=config.groups)
    blocks = tuple(
        BlockSpec(prefix=f"l{index}", mixer=_mixer_spec(layer.mixer, config.width, config.eps), feed_forward=_feed_forward_spec(layer.mlp, config.width),
                  mixer_norm=norm, feed_forward_norm=None, kind="parallel", residual_scale=config.residual_mult)
        for index, layer in enumerate(config.layers)
    )
    # Layers whose mixers keep the same thing share a cache group with a cache layer each; so does everything that a mixer keeps
    # beside its own cache (the other side's state, the convolutions' tails, the shifted input), role by role.  A layer that reads
    # another's keys and values is given that layer's group and cache layer and writes nothing there.
    schedule, counters, names, placed = [], {}, {}, {}

    def place(need_key, label):
        group = names.setdefault(need_key, f"{label}.{len(names)}")
        layer = counters.get(group, 0)
        counters[group] = layer + 1
        return group, layer

    for index, (block, layer) in enumerate(zip(blocks, config.layers)):
        mixer, extra, writes = block.mixer, [], True
        if mixer.kind == "masked_attention":
            source = layer.mixer.kv_from
            if source is None:
                group, cache_layer = place(("keys", mixer.n_kv_heads, mixer.dim, mixer.value_dim), "keys")
            else:
                (group, cache_layer), writes = placed[source], False
            if mixer.taps > 1:
                channels = mixer.n_heads * mixer.dim + (mixer.n_kv_heads * (mixer.dim + mixer.value_dim) if mixer.own_keys else 0)
                extra.append(("taps", *place(("taps", mixer.taps, channels), "taps")))
        elif mixer.kind == "channel_decay_memory":
            group, cache_layer = place(("memory", mixer.n_heads, mixer.key_dim), "memory")
            extra.append(("shift", *place(("shift", config.width), "shift")))
        else:
            left, right = mixer.left, mixer.right
            group, cache_layer = place(("keys", left.n_kv_heads, left.dim, left.value_dim), "keys")
            extra.append(("right", *place(("delta", right.n_heads, right.key_dim, right.value_dim), "delta")))
            if right.taps > 1:
                channels = 2 * right.n_key_heads * right.key_dim + right.n_heads * right.value_dim
                extra.append(("right.taps", *place(("taps", right.taps, channels), "taps")))
        placed[index] = (group, cache_layer)
        schedule.append(ScheduleEntry(layer=index, cache_group=group, cache_layer=cache_layer, writes_cache=writes, extra_cache=tuple(extra)))
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=config.vocab, hidden=config.width, max_positions=MAX_POSITIONS, embedding_name="embed",
        blocks=blocks, schedule=tuple(schedule), final_norm=norm, final_norm_name="final.norm", head_name="head", tie_head=False,
        declared_dtype=config.declared_dtype, residual_dtype="float32", logit_scale=config.logit_scale,
    )


register_architecture(ARCHITECTURE, MODEL_TYPE, NugolornConfig.from_json, build_nugolorn_spec, storage_dtype="bfloat16", complete_config=sizes_from_tensors)
