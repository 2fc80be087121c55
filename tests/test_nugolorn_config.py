"""Nugolorn on the host: its configuration, the blocks and schedule built from it, what its cache keeps, sizes that only tensors'
shapes give, and the plain statement against itself and against closed forms."""
import copy
import math

import pytest
import torch

import nugolorn_models as nm
import plain_nugolorn as plain
from tau_rs_b200.config import InvalidConfig, NugolornConfig
from tau_rs_b200.config.metadata import metadata_from_json
from tau_rs_b200.config.nugolorn import sizes_from_tensors
from tau_rs_b200.config.registry import architecture_for, spec_from_config_json
from tau_rs_b200.parts import DecoderModel

ALL = (nm.MIXED, nm.ODD, nm.MANY_GROUPS, nm.PEAKY, nm.HEADY, nm.LONG_MEMORY, *nm.ONLY.values())


def test_the_architecture_is_registered_and_stores_bfloat16():
    metadata = metadata_from_json(nm.MIXED)
    assert (metadata.architecture, metadata.model_type, metadata.declared_dtype) == ("Nugolorn", "nugolorn", None)
    assert architecture_for(nm.MIXED).storage_dtype == "bfloat16"


def test_every_size_and_constant_is_read_from_the_configuration():
    config = NugolornConfig.from_json(nm.MIXED)
    assert (config.vocab, config.width, config.eps, config.groups, config.residual_mult, config.logit_scale) == (211, 96, 1e-5, 3, 0.6, 0.5)
    first, second, third, fourth = config.layers[:4]
    mixer = first.mixer
    assert (mixer.heads, mixer.kv_heads, mixer.dim, mixer.vdim, mixer.scale, mixer.taps, mixer.rot_base, mixer.rot_dims, mixer.kv_from) == (4, 2, 16, 24, 0.25, 4, 5000.0, 8, None)
    assert (second.mixer.heads, second.mixer.dim, second.mixer.decay_rank) == (3, 16, 6)
    assert (second.mlp.kind, second.mlp.experts, second.mlp.identity, second.mlp.top, second.mlp.expert_ff) == ("moe", 5, 2, 3, 40)
    left, right = third.mixer.left, third.mixer.right
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.scale, left.temperature) == (4, 2, 16, 24, 0.25, (0.4, 16))
    assert (right.heads, right.kv_heads, right.dim, right.vdim, right.taps, right.decay_rank, right.gate_rank) == (4, 2, 16, 24, 3, 5, 7)
    assert fourth.mixer.kv_from == 0 and fourth.mixer.heads == 6 and first.mlp.ff == 72 and config.layers[4].mlp is None
    odd = NugolornConfig.from_json(nm.ODD)
    assert odd.layers[3].mixer.taps == 0 and odd.layers[3].mixer.rot_dims == 0 and odd.layers[4].mixer.left.temperature is None
    # What a configuration may leave out has the value that changes nothing.
    bare = copy.deepcopy(nm.ONLY["wkv"])
    del bare["residual_mult"], bare["logit_scale"], bare["norm"]["groups"]
    bare = NugolornConfig.from_json(bare)
    assert (bare.residual_mult, bare.logit_scale, bare.groups) == (1.0, 1.0, 1)


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="mamba1"), "type must be one of"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"]["right"].pop("conv"), "'conv'"),
    (lambda c: c["layers"][1]["mixer"].update(dim=0), "'dim'"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=8), "exceeds"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(dim=8), "kv_from"),
    (lambda c: c["layers"][7]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].pop("decay_rank"), "decay_rank"),
    (lambda c: c["layers"][2]["mixer"]["right"].pop("gate_rank"), "gate_rank"),
    (lambda c: c["norm"].update(groups=5), "norm.groups"),
    (lambda c: c.pop("norm"), "'norm'"),
])
def test_a_configuration_that_does_not_fit_is_refused_by_name(change, message):
    raw = copy.deepcopy(nm.MIXED)
    change(raw)
    with pytest.raises(InvalidConfig, match=message):
        NugolornConfig.from_json(raw)


def test_sizes_that_only_tensor_shapes_give():
    raw = copy.deepcopy(nm.MIXED)
    shapes = {name: tuple(value.shape) for name, value in nm.weights(nm.MIXED, 1).items()}
    del raw["layers"][1]["mixer"]["decay_rank"], raw["layers"][2]["mixer"]["right"]["decay_rank"], raw["layers"][6]["mixer"]["right"]["gate_rank"]
    completed = sizes_from_tensors(raw, shapes)
    assert NugolornConfig.from_json(completed) == NugolornConfig.from_json(nm.MIXED)
    assert "decay_rank" not in raw["layers"][1]["mixer"]                           # the caller's dictionary is left as it was
    given = copy.deepcopy(nm.MIXED)
    given["layers"][1]["mixer"]["decay_rank"] = 2                                  # what config.json says is not overwritten
    assert sizes_from_tensors(given, shapes)["layers"][1]["mixer"]["decay_rank"] == 2


def test_blocks_schedule_and_cache_groups():
    spec = spec_from_config_json(nm.MIXED)
    assert spec.residual_dtype == "float32" and not spec.tie_head and spec.logit_scale == 0.5
    assert [block.kind for block in spec.blocks] == ["parallel"] * 8 and all(block.residual_scale == 0.6 for block in spec.blocks)
    assert all(block.mixer_norm.groups == 3 for block in spec.blocks) and spec.final_norm.groups == 3
    assert [block.mixer.kind for block in spec.blocks] == ["masked_attention", "channel_decay_memory", "side_by_side", "masked_attention", "masked_attention",
                                                           "channel_decay_memory", "side_by_side", "masked_attention"]
    first, shared = spec.blocks[0].mixer, spec.blocks[3].mixer
    assert first.weights == "sigmoid" and first.gate == "head" and first.bias and first.taps == 4 and first.own_keys and not first.sink and not first.distance_bias
    assert not shared.own_keys and shared.n_heads == 6
    side = spec.blocks[2].mixer
    assert side.join == "normed" and (side.left_scale, side.right_scale) == (0.5, 0.5) and side.left.distance_bias and side.left.gate == "element"
    assert side.left.temperature == (0.4, 16) and side.left.position is None and side.left.weights == "softmax"
    assert side.right.decay == "channel" and side.right.gate_activation == "sigmoid" and (side.right.decay_rank, side.right.gate_rank) == (5, 7)
    experts = spec.blocks[1].feed_forward
    assert experts.score == "softmax" and experts.correction and not experts.renormalize and experts.identity == 2 and experts.shared is None
    assert spec.blocks[4].feed_forward is None and spec.blocks[0].feed_forward.activation == "silu"
    # A layer that reads another's keys names that layer's place in the cache and writes nothing there; nothing else is shared.
    by_layer = {entry.layer: entry for entry in spec.schedule}
    assert (by_layer[3].cache_group, by_layer[3].cache_layer, by_layer[3].writes_cache) == (by_layer[0].cache_group, by_layer[0].cache_layer, False)
    assert (by_layer[7].cache_group, by_layer[7].cache_layer, by_layer[7].writes_cache) == (by_layer[4].cache_group, by_layer[4].cache_layer, False)
    places = set()
    for entry in spec.schedule:
        for place in ([(entry.cache_group, entry.cache_layer)] if entry.writes_cache else []) + [(group, layer) for _, group, layer in entry.extra_cache]:
            assert place not in places
            places.add(place)
    assert [role for role, _, _ in by_layer[0].extra_cache] == ["taps"] and [role for role, _, _ in by_layer[1].extra_cache] == ["shift"]
    assert [role for role, _, _ in by_layer[2].extra_cache] == ["right", "right.taps"]
    groups = DecoderModel(spec, torch.float32, "cpu").cache_groups()
    rows = sorted((need.row_width, need.window, need.chunk, layers) for need, layers in groups.values() if need.kind == "rows")
    assert rows == [(1 * (8 + 40), None, None, 1), (2 * (16 + 24), None, None, 2), (3 * (8 + 40), None, None, 1)]
    states = sorted((need.state_shape, layers) for need, layers in groups.values() if need.kind == "state")
    assert states == sorted([((3, 4 * 16 + 2 * 40), 1), ((3, 6 * 16), 1), ((1, 2 * 8 + 48), 1), ((1, 4 * 8), 1),          # the attention layers' tails
                             ((3 * 16 * 16,), 1), ((2 * 24 * 24,), 1), ((96,), 2),                                         # memories and shifted inputs
                             ((4 * 24 * 16,), 1), ((6 * 8 * 24,), 1), ((2, 2 * 2 * 16 + 4 * 24), 1), ((1, 2 * 2 * 24 + 6 * 8), 1)])


def test_keys_and_values_as_wide_as_ordinary_heads_lie_in_pages_of_heads():
    groups = DecoderModel(spec_from_config_json(nm.HEADY), torch.float32, "cpu").cache_groups()
    assert not [need for need, _ in groups.values() if need.kind == "rows"]
    assert sorted((need.n_kv_heads, need.head_dim, layers) for need, layers in groups.values() if need.kind == "kv") == [(1, 64, 1), (2, 128, 1)]


def test_one_tap_or_none_keeps_no_tail():
    spec = spec_from_config_json(nm.ODD)
    assert spec.schedule[0].extra_cache == () and spec.schedule[3].extra_cache == ()
    assert [role for role, _, _ in spec.schedule[2].extra_cache] == ["right"] and [role for role, _, _ in spec.schedule[5].extra_cache] == ["taps"]


def test_the_model_asks_for_exactly_the_tensors_of_the_design():
    for cfg in ALL:
        wanted = DecoderModel.tensor_specs_of(spec_from_config_json(cfg))
        made = nm.weights(cfg, 1)
        assert set(wanted) == set(made)
        for name, value in made.items():
            assert tuple(wanted[name].shape) == tuple(value.shape), name


def _double(values):
    return {name: value.double() for name, value in values.items()}


def test_the_plain_statement_is_causal():
    for cfg in (nm.MIXED, nm.ODD):
        values = _double(nm.weights(cfg, 3))
        tokens = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(5)).tolist()
        whole = plain.forward(tokens, values, cfg)
        assert torch.allclose(plain.forward(tokens[:41], values, cfg), whole[:41], atol=1e-9)


def test_the_plain_mechanisms_against_closed_forms():
    generator = torch.Generator().manual_seed(9)
    rand = lambda *shape: torch.randn(*shape, dtype=torch.float64, generator=generator)
    # One group is the ordinary RMS norm; as many groups as elements leave the signs times the weight.
    x, w = rand(4, 12), rand(12)
    assert torch.allclose(plain.grouped_rms_norm(x, w, 1, 1e-6), x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w, atol=1e-12)
    assert torch.allclose(plain.grouped_rms_norm(x, w, 12, 0.0), torch.sign(x) * w, atol=1e-12)
    pieces = plain.grouped_rms_norm(x, torch.ones(12, dtype=torch.float64), 3, 0.0).reshape(4, 3, 4)
    assert torch.allclose((pieces * pieces).mean(-1), torch.ones(4, 3, dtype=torch.float64), atol=1e-12)
    # Sigmoid weights: the first token sees itself alone; a far offset below zero silences a head.
    q, k, v = rand(9, 2, 4), rand(9, 1, 4), rand(9, 1, 3)
    out = plain.sigmoid_attention(q, k, v, 0.5, torch.tensor([0.3, -50.0], dtype=torch.float64))
    assert torch.allclose(out[0, 0], torch.sigmoid((q[0, 0] * k[0, 0]).sum() * 0.5 + 0.3) * v[0, 0], atol=1e-12)
    assert out[:, 1].abs().max() < 1e-12
    by_hand = sum(torch.sigmoid((q[5, 0] * k[j, 0]).sum() * 0.5 + 0.3) * v[j, 0] for j in range(6))
    assert torch.allclose(out[5, 0], by_hand, atol=1e-12)
    # The distance bias: with r1 = 0 a plain causal softmax; with equal scores the weights fall as (1 + r2 d)^-r1.
    zeros, ones = torch.zeros(2, dtype=torch.float64), torch.ones(2, dtype=torch.float64)
    plain_softmax = plain.distance_softmax_attention(q, k, v, 0.5, zeros, ones)
    scores = (q[:, 0] @ k[:, 0].T) * 0.5 + torch.triu(torch.full((9, 9), -math.inf, dtype=torch.float64), 1)
    assert torch.allclose(plain_softmax[:, 0], torch.softmax(scores, -1) @ v[:, 0], atol=1e-12)
    flat = plain.distance_softmax_attention(torch.zeros(9, 2, 4, dtype=torch.float64), k, v, 0.5, 2.0 * ones, 0.5 * ones)
    weights = (1.0 + 0.5 * torch.arange(8, -1, -1, dtype=torch.float64)) ** -2.0
    assert torch.allclose(flat[8, 0], (weights / weights.sum()) @ v[:, 0], atol=1e-12)
    # The delta rule with beta = 1, no decay and orthonormal keys stores each value under its key; a decay of zero on every
    # channel forgets everything before the token.
    keys = torch.linalg.qr(rand(6, 6)).Q[:, None, :]
    values = rand(6, 1, 4)
    one = torch.ones(6, 1, dtype=torch.float64)
    assert torch.allclose(plain.channel_gated_delta_rule(keys, keys, values, one, torch.ones(6, 1, 6, dtype=torch.float64)), values, atol=1e-12)
    forgetful = plain.channel_gated_delta_rule(rand(6, 1, 6), keys, values, one, torch.zeros(6, 1, 6, dtype=torch.float64))
    probe = plain.channel_gated_delta_rule(keys, keys, values, one, torch.zeros(6, 1, 6, dtype=torch.float64))
    assert torch.allclose(probe, values, atol=1e-12) and forgetful.shape == values.shape
    # A decay on one channel alone touches only what was written along that channel.
    basis = torch.eye(3, dtype=torch.float64)[:, None, :]
    decay = torch.ones(3, 1, 3, dtype=torch.float64)
    decay[2, 0, 0] = 0.25
    stored = rand(3, 1, 2)
    read = plain.channel_gated_delta_rule(torch.ones(3, 1, 3, dtype=torch.float64), basis, stored, torch.ones(3, 1, dtype=torch.float64), decay)
    assert torch.allclose(read[2, 0], 0.25 * stored[0, 0] + stored[1, 0] + stored[2, 0], atol=1e-12)
    # The matrix memory: the first token reads only its own write, weighed by the bonus; the second sees the first undecayed.
    r, k2, v2, w2, bonus = rand(3, 1, 4), rand(3, 1, 4), rand(3, 1, 2), torch.rand(3, 1, 4, dtype=torch.float64, generator=generator), rand(1, 4)
    out = plain.wkv_recurrence(r, k2, v2, w2, bonus)
    assert torch.allclose(out[0, 0], (r[0, 0] * bonus[0] * k2[0, 0]).sum() * v2[0, 0], atol=1e-12)
    second = (r[1, 0] * k2[0, 0]).sum() * v2[0, 0] + (r[1, 0] * bonus[0] * k2[1, 0]).sum() * v2[1, 0]
    assert torch.allclose(out[1, 0], second, atol=1e-12)
    third = (r[2, 0] * w2[1, 0] * k2[0, 0]).sum() * v2[0, 0] + (r[2, 0] * k2[1, 0]).sum() * v2[1, 0] + (r[2, 0] * bonus[0] * k2[2, 0]).sum() * v2[2, 0]
    assert torch.allclose(out[2, 0], third, atol=1e-12)
    # A convolution of one tap is a scale; of three taps it reaches two rows back and sees zeros before the start.
    x, taps = rand(5, 3), rand(3, 3)
    assert torch.allclose(plain.causal_convolution(x, taps[:, :1]), x * taps[:, 0], atol=1e-12)
    assert torch.allclose(plain.causal_convolution(x, taps)[1], taps[:, 2] * x[1] + taps[:, 1] * x[0], atol=1e-12)


def test_identity_experts_return_what_they_read():
    generator = torch.Generator().manual_seed(4)
    width = 8
    h = torch.randn(5, width, dtype=torch.float64, generator=generator)
    mlp = {"kind": "moe", "router": {"experts": 1, "identity": 2, "top": 2}, "expert": {"ff": 4}}
    weights = {"m.router": torch.zeros(3, width, dtype=torch.float64), "m.correction": torch.tensor([-1.0, 0.5, 0.2], dtype=torch.float64),
               "m.e0.gate": torch.randn(4, width, dtype=torch.float64, generator=generator), "m.e0.up": torch.randn(4, width, dtype=torch.float64, generator=generator),
               "m.e0.down": torch.randn(width, 4, dtype=torch.float64, generator=generator)}
    # Equal scores of one third; the correction keeps the expert with tensors out: two identity experts return 2/3 of the input.
    assert torch.allclose(plain.routed_feed_forward(h, weights, "m", mlp), h * (2.0 / 3.0), atol=1e-12)
    weights["m.correction"] = torch.tensor([1.0, 0.5, 0.2], dtype=torch.float64)
    expected = (plain.gated_feed_forward(h, weights, "m.e0") + h) / 3.0            # the correction chooses, the score alone weighs
    assert torch.allclose(plain.routed_feed_forward(h, weights, "m", mlp), expected, atol=1e-12)
