"""Pegurax on the host: its configuration, the blocks and schedule built from it, what its cache keeps and gives back, the rotation's
frequencies, and the plain statement against itself (prompts cut by hand, a chunk that covers everything)."""
import copy
import math

import pytest
import torch

import pegurax_models as pm
import plain_pegurax as plain
from tau_rs_b200.cache import SequenceCache
from tau_rs_b200.config import InvalidConfig, PeguraxConfig, ScaledRotationSpec
from tau_rs_b200.config.metadata import metadata_from_json
from tau_rs_b200.config.registry import architecture_for, spec_from_config_json
from tau_rs_b200.parts import CacheNeed, DecoderModel
from tau_rs_b200.parts.registry import build

ALL = (pm.MIXED, pm.ODD, pm.PEAKY, pm.EDGY, pm.LONG_MEMORY)


def test_the_architecture_is_registered_and_stores_bfloat16():
    metadata = metadata_from_json(pm.MIXED)
    assert (metadata.architecture, metadata.model_type, metadata.declared_dtype) == ("Pegurax", "pegurax", None)
    assert architecture_for(pm.MIXED).storage_dtype == "bfloat16"


def test_every_size_and_constant_is_read_from_the_configuration():
    config = PeguraxConfig.from_json(pm.MIXED)
    assert (config.vocab, config.width, config.eps, config.embedding_scale) == (211, 96, 1e-5, 0.75)
    first, second, third = config.layers[0], config.layers[1], config.layers[2]
    left, right = first.mixer.left, first.mixer.right
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.chunk, left.rot_dims, left.rot_base, left.scale) == (4, 2, 16, 24, 37, 8, 5000.0, 0.25)
    assert (left.rot_scaling.factor, left.rot_scaling.original, left.rot_scaling.fast, left.rot_scaling.slow) == (4.0, 64.0, 16.0, 2.0)
    assert (right.heads, right.kv_heads, right.dim, right.vdim, right.taps) == (4, 2, 16, 24, 4)
    assert (first.mixer.left_scale, first.mixer.right_scale) == (0.7, 1.3)
    assert (second.mixer.inner, second.mixer.states, second.mixer.dt_rank, second.mixer.taps) == (80, 8, 6, 3)
    assert (second.mlp.kind, second.mlp.experts, second.mlp.top, second.mlp.expert_ff) == ("moe", 6, 2, 40)
    assert first.mlp.kind == "dense" and first.mlp.ff == 72 and third.mlp is None and third.mixer.left.rot_scaling is None


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="attention"), "type must be one of"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("conv"), "'conv'"),
    (lambda c: c["layers"][1]["mixer"].update(state=0), "'state'"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "exceeds"),
    (lambda c: c.pop("embedding"), "'embedding'"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "'left_scale'"),
])
def test_a_configuration_that_does_not_fit_is_refused_by_name(change, message):
    raw = copy.deepcopy(pm.MIXED)
    change(raw)
    with pytest.raises(InvalidConfig, match=message):
        PeguraxConfig.from_json(raw)


def test_blocks_schedule_and_cache_groups():
    spec = spec_from_config_json(pm.MIXED)
    assert spec.residual_dtype == "float32" and spec.tie_head and spec.embedding_scale == 0.75
    assert [block.kind for block in spec.blocks] == ["sandwich"] * 5
    assert [block.mixer.kind for block in spec.blocks] == ["side_by_side", "selective_scan", "side_by_side", "selective_scan", "selective_scan"]
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].feed_forward_norm is None and spec.blocks[2].feed_forward_post_norm is None
    assert spec.blocks[0].feed_forward.activation == "relu" and spec.blocks[1].feed_forward.weigh == "input" and not spec.blocks[1].feed_forward.renormalize
    left = spec.blocks[0].mixer.left
    assert left.sink and left.chunk == 37 and left.window is None and left.qk_norm == "projection"
    places = set()
    for entry in spec.schedule:
        for place in [(entry.cache_group, entry.cache_layer)] + [(group, layer) for _, group, layer in entry.extra_cache]:
            assert place not in places                       # nothing is kept in one place by two layers
            places.add(place)
    assert [role for role, _, _ in spec.schedule[0].extra_cache] == ["right", "right.taps"] and [role for role, _, _ in spec.schedule[1].extra_cache] == ["taps"]
    groups = DecoderModel(spec, torch.float32, "cpu").cache_groups()
    rows = sorted((need.row_width, need.chunk, need.window, layers) for need, layers in groups.values() if need.kind == "rows")
    assert rows == [(2 * (16 + 24), 37, None, 1), (3 * (8 + 40), 70, None, 1)]
    states = sorted((need.state_shape, layers) for need, layers in groups.values() if need.kind == "state")
    assert states == sorted([((4 * 24 * 16,), 1), ((6 * 8 * 24,), 1), ((3, 2 * 2 * 16 + 4 * 24), 1), ((1, 2 * 2 * 24 + 6 * 8), 1),
                             ((80 * 8,), 1), ((48 * 16,), 1), ((64 * 4,), 1), ((2, 80), 1), ((3, 48), 1), ((1, 64), 1)])


def test_keys_and_values_as_wide_as_ordinary_heads_lie_in_pages_of_heads():
    groups = DecoderModel(spec_from_config_json(pm.HEADY), torch.float32, "cpu").cache_groups()
    assert not [need for need, _ in groups.values() if need.kind == "rows"]
    heads = sorted((need.n_kv_heads, need.head_dim, need.chunk, need.window, layers) for need, layers in groups.values() if need.kind == "kv")
    assert heads == [(1, 64, 96, None, 1), (2, 128, 50, None, 1)]


def test_one_tap_keeps_no_tail():
    spec = spec_from_config_json(pm.ODD)
    assert [role for role, _, _ in spec.schedule[0].extra_cache] == ["right"] and spec.schedule[1].extra_cache == ()


def test_the_model_asks_for_exactly_the_tensors_of_the_design():
    for cfg in ALL:
        wanted = DecoderModel.tensor_specs_of(spec_from_config_json(cfg))
        made = pm.weights(cfg, 1)
        assert set(wanted) == set(made)
        for name, value in made.items():
            assert tuple(wanted[name].shape) == tuple(value.shape), name


def test_the_rotations_frequencies():
    for rot in (pm.softmax_side()["rot"], pm.softmax_side(rot_dims=16, scaling=pm.yarn(8.0, 512, 32.0, 1.0))["rot"], pm.softmax_side(scaling=None)["rot"],
                pm.softmax_side(dim=64, rot_dims=64, base=40000.0, scaling=pm.yarn(2.0, 20, 3.0, 1.5))["rot"]):
        scaling = rot.get("scaling") or {}
        part = build("position", ScaledRotationSpec(rotary_dim=rot["dims"], theta=rot["base"], factor=scaling.get("factor"), original=scaling.get("original", 0.0),
                                                    fast=scaling.get("fast", 0.0), slow=scaling.get("slow", 0.0)), device="cpu")
        found, magnitude = part.values()
        wanted, wanted_magnitude = plain.scaled_frequencies(rot)
        assert found == pytest.approx(wanted, rel=1e-12) and magnitude == pytest.approx(wanted_magnitude, rel=1e-12)
    # The blend by hand for one case: 8 pairs, base 100, factor 4, 64 original positions, between 16 turns and 2.
    dims, base = 16, 100.0
    index = lambda turns: dims * math.log(64 / (2 * math.pi * turns)) / (2 * math.log(base))
    low, high = max(math.floor(index(16.0)), 0), min(math.ceil(index(2.0)), dims - 1)
    assert (low, high) == (0, 3)
    frequencies, magnitude = plain.scaled_frequencies({"dims": dims, "base": base, "scaling": pm.yarn(4.0, 64, 16.0, 2.0)})
    assert frequencies[0] == 1.0 and frequencies[7] == pytest.approx(base ** (-14 / 16) / 4) and frequencies[1] == pytest.approx(base ** (-2 / 16) * (1 - 1 / 3 + 1 / 12))
    assert magnitude == pytest.approx(0.1 * math.log(4.0) + 1.0)


def test_a_chunked_cache_gives_back_the_pages_before_the_newest_chunk():
    groups = {"rows": (CacheNeed("rows", row_width=8, chunk=100), 1), "state": (CacheNeed("state", state_shape=(3,)), 1)}
    cache = SequenceCache(groups, 64 * 4, 1 << 20, torch.float32, "cpu")
    slot, other = cache.open(), cache.open()
    cache.reserve(other, 10)
    cache.advance(other, 10)
    length = 0
    for count in [50, 49, 1, 1, 64, 35, 1, 99, 1, 1, 120, 3]:
        cache.reserve(slot, length + count)
        length += count
        cache.advance(slot, length)
        cache.check()
        first_needed = length // 100 * 100 // 64                         # the page of the first position that position `length` sees
        assert cache.kv["rows"].released[slot] == first_needed
        assert len(cache.kv["rows"].held[slot]) == -(-length // 64) - first_needed
        assert cache.kv["rows"].tokens_read(length) == length % 100
    assert length > 64 * 4                                               # the sequence outgrew the whole cache
    cache.close(slot)
    cache.close(other)
    cache.check()
    assert cache.kv["rows"].pool.in_use == 0


def _double(values):
    return {name: value.double() for name, value in values.items()}


def test_the_plain_statement_is_causal_and_its_chunks_start_at_position_zero():
    cfg = pm.MIXED
    values = _double(pm.weights(cfg, 3))
    tokens = torch.randint(0, cfg["vocab"], (90,), generator=torch.Generator().manual_seed(5)).tolist()
    whole = plain.forward(tokens, values, cfg)
    assert torch.allclose(plain.forward(tokens[:41], values, cfg), whole[:41], atol=1e-9)
    # A chunk that covers everything is plain causal attention with a sink.
    q, k, v = (torch.randn(50, 8, dtype=torch.float64, generator=torch.Generator().manual_seed(seed)) for seed in (1, 2, 3))
    everything = plain.chunked_sink_attention(q, k, v, 0.4, 1000)
    scores = (q @ k.T) * 0.4 + torch.triu(torch.full((50, 50), float("-inf"), dtype=torch.float64), 1)
    weights = torch.exp(scores)
    assert torch.allclose(everything, (weights / (1.0 + weights.sum(-1, keepdim=True))) @ v, atol=1e-12)
    chunked = plain.chunked_sink_attention(q, k, v, 0.4, 7)
    assert torch.allclose(chunked[7:14], plain.chunked_sink_attention(q[7:14], k[7:14], v[7:14], 0.4, 7), atol=1e-12)
    assert not torch.allclose(chunked[8], everything[8], atol=1e-3)


def test_the_plain_recurrences_against_their_closed_forms():
    generator = torch.Generator().manual_seed(9)
    # The delta rule with beta = 1, no decay and orthonormal keys stores each value under its key.
    keys = torch.linalg.qr(torch.randn(6, 6, dtype=torch.float64, generator=generator)).Q
    values = torch.randn(6, 4, dtype=torch.float64, generator=generator)
    out = plain.gated_delta_rule(keys, keys, values, torch.ones(6, dtype=torch.float64), torch.ones(6, dtype=torch.float64))
    assert torch.allclose(out, values, atol=1e-12)
    # With a decay g and beta = 1 the same key twice returns the second value, and the first one's trace is gone.
    twice = plain.gated_delta_rule(keys[[0, 0]], keys[[0, 0]], values[:2], torch.ones(2, dtype=torch.float64), torch.tensor([0.5, 0.5], dtype=torch.float64))
    assert torch.allclose(twice[1], values[1], atol=1e-12)
    # A convolution of one tap is a scale; of three taps it reaches two rows back and sees zeros before the start.
    x = torch.randn(5, 3, dtype=torch.float64, generator=generator)
    taps = torch.randn(3, 3, dtype=torch.float64, generator=generator)
    assert torch.allclose(plain.causal_convolution(x, taps[:, :1]), x * taps[:, 0], atol=1e-12)
    by_hand = taps[:, 2] * x[1] + taps[:, 1] * x[0]
    assert torch.allclose(plain.causal_convolution(x, taps)[1], by_hand, atol=1e-12)
