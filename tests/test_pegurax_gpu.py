"""Pegurax on the GPU against the plain statement in `plain_pegurax.py`: each mechanism's kernels alone, then whole models: whole
prompts, single tokens, portions, unequal batches, slots, pages and states that are used again, chunk edges and page borders, keys
far back, long decoding, odd sizes, greedy generation through `generate()`, the command line and the trace replay."""
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import pegurax_models as pm
import plain_pegurax as plain
from helpers import relative_error, run_batched, run_tail_stepwise, run_whole
from tau_rs_b200 import Engine, StepEntry, generate, load_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOLERANCE = {"float32": 5e-5, "bfloat16": 4e-2}
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEVICE = "cuda"


def close(found, wanted, dtype) -> bool:
    """float32: every logit within 5e-5 of the largest.  bfloat16 (the plain statement rounds nothing): half of the positions within
    2e-2 of the largest logit and all but one in ten (or two) within 6e-2; where two experts were a close call the library and the
    plain statement may choose differently at a position, which says nothing about either (the float32 runs pin every choice)."""
    if dtype == "float32":
        return relative_error(found, wanted) < TOLERANCE[dtype]
    rows = (found.double() - wanted.double()).abs().amax(dim=-1) / wanted.double().abs().max()
    return float(rows.median()) < 2e-2 and int((rows >= 6e-2).sum()) <= max(2, rows.numel() // 10)


def tokens_for(cfg, count, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=count).tolist()


_PLAIN = {}


def plain_logits(cfg, values, tokens):
    key = (id(values), tuple(tokens))
    if key not in _PLAIN:
        _PLAIN[key] = plain.forward(tokens, {name: value.double() for name, value in values.items()}, cfg).float()
    return _PLAIN[key]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("pegurax")
    made = {}
    for name, cfg, seed, slow in (("mixed", pm.MIXED, 11, False), ("odd", pm.ODD, 12, False), ("peaky", pm.PEAKY, 14, False), ("edgy", pm.EDGY, 15, False), ("heady", pm.HEADY, 17, False),
                                  ("long_memory", pm.LONG_MEMORY, 16, True)):
        folder = str(root / name)
        made[name] = (folder, cfg, pm.write_model(folder, cfg, seed, slow_decay=slow))
    return made


def engine_of(models, name, dtype, max_tokens=1024):
    folder, cfg, values = models[name]
    return Engine(load_model(folder, dtype, "gpu"), max_tokens), cfg, values


def on_device(tensor, dtype=torch.float32):
    return tensor.to(DEVICE, dtype).contiguous()


def as_ints(values):
    return torch.tensor(np.asarray(values, dtype=np.int32), device=DEVICE)


def packed_step(runs, slots):
    """The metadata of a step in which sequence i brings `runs[i]` tokens and sits in cache slot `slots[i]`."""
    bounds = np.concatenate([[0], np.cumsum(runs)]).astype(np.int32)
    token_seq = np.concatenate([np.full(count, index, dtype=np.int32) for index, count in enumerate(runs)])
    return SimpleNamespace(n_seqs=len(runs), token_seq=as_ints(token_seq), cu_seqlens=as_ints(bounds), seq_slot=as_ints(slots),
                           all_single=all(count == 1 for count in runs))


STEPS = ([1, 9, 2], [1, 1, 1], [1, 1, 1], [2, 1, 6], [1, 1, 1], [5, 2, 1], [40, 3, 1], [150, 1, 67])      # runs of three sequences, step by step


# ---- each mechanism's kernels alone -----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps, biased, silu", [(1, False, True), (2, True, True), (4, False, True), (4, True, False), (7, True, True)])
def test_short_convolutions_carry_their_last_inputs_from_step_to_step(dtype, taps, biased, silu):
    """Three sequences in slots 5, 0 and 2 of a state that held other values; runs shorter and longer than the tail: every step
    equals the plain convolution of the whole sequence so far, read from a column range and written into one."""
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(taps)
    width, slots = 52, [5, 0, 2]
    weight = torch.randn(width, taps, dtype=torch.float64)
    bias = torch.randn(width, dtype=torch.float64) if biased else None
    state = torch.randn(7, max(taps - 1, 1), width, device=DEVICE)[:, : taps - 1].contiguous() if taps > 1 else None
    if state is not None:
        state[slots] = 0.0          # a sequence starts from zeros, as the cache leaves a slot
    history = [torch.zeros(0, width, dtype=torch.float64) for _ in slots]
    for runs in STEPS:
        new = [torch.randn(count, width).to(TORCH[dtype]).double() for count in runs]
        wide = torch.zeros(sum(runs), width + 9, dtype=TORCH[dtype], device=DEVICE)
        wide[:, 4 : 4 + width] = torch.cat(new).to(DEVICE, TORCH[dtype])
        out = torch.zeros(sum(runs), width + 3, dtype=torch.float32, device=DEVICE)
        kernels.short_conv(wide[:, 4 : 4 + width], on_device(weight.T), None if bias is None else on_device(bias), state, packed_step(runs, slots),
                           out[:, 3:], silu=silu, update=True)
        wanted = []
        for index, rows in enumerate(new):
            history[index] = torch.cat([history[index], rows])
            mixed = plain.causal_convolution(history[index], weight, bias)
            wanted.append((plain.silu(mixed) if silu else mixed)[-rows.shape[0] :])
        assert relative_error(out[:, 3:].cpu(), torch.cat(wanted)) < 2e-6
        assert float(out[:, :3].abs().max()) == 0.0


def plain_delta_heads(q, k, v, pre_beta, pre_step, a_log, dt_bias, heads, key_heads, dim, vdim):
    """The plain gated delta rule of one sequence from the convolutions' outputs on: unit vectors, gates, recurrence."""
    tokens = q.shape[0]
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k, v = unit(q.view(tokens, key_heads, dim)) * dim ** -0.5, unit(k.view(tokens, key_heads, dim)), v.view(tokens, heads, vdim)
    beta, decay = torch.sigmoid(pre_beta), torch.exp(-torch.exp(a_log) * plain.softplus(pre_step + dt_bias))
    out = torch.zeros((tokens, heads, vdim), dtype=torch.float64)
    for head in range(heads):
        group = head // (heads // key_heads)
        out[:, head] = plain.gated_delta_rule(q[:, group], k[:, group], v[:, head], beta[:, head], decay[:, head])
    return out.reshape(tokens, heads * vdim)


@pytest.mark.parametrize("heads, key_heads, dim, vdim", [(4, 2, 16, 24), (1, 1, 20, 70), (3, 3, 6, 34), (2, 1, 100, 10), (6, 2, 32, 32), (2, 2, 128, 64), (8, 4, 64, 130)])
def test_the_gated_delta_rule_carries_its_state_from_step_to_step(heads, key_heads, dim, vdim):
    """Three sequences in slots out of order, runs of one and of many tokens, over seven steps: every step continues the plain
    recurrence of the whole sequence.  The decays are slow, so the first tokens still weigh in the last."""
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(dim + vdim)
    slots, k_width, v_width = [3, 0, 1], key_heads * dim, heads * vdim
    a_log, dt_bias = -3.0 + 0.5 * torch.randn(heads, dtype=torch.float64), 0.5 * torch.randn(heads, dtype=torch.float64)
    state = torch.randn(5, heads * vdim * dim, device=DEVICE)
    state[slots] = 0.0
    history = [[torch.zeros(0, width, dtype=torch.float64) for width in (k_width, k_width, v_width, heads, heads)] for _ in slots]
    for runs in STEPS:
        tokens = sum(runs)
        new = [[torch.randn(count, width).double() for width in (k_width, k_width, v_width, heads, heads)] for count in runs]
        rows = on_device(torch.cat([torch.cat(pieces[:3], dim=1) for pieces in new]))
        pre = on_device(torch.cat([torch.cat(pieces[3:], dim=1) for pieces in new]))
        gates = torch.empty((tokens, heads, 2), dtype=torch.float32, device=DEVICE)
        kq = torch.empty((tokens, key_heads), dtype=torch.float32, device=DEVICE)
        kernels.delta_prepare(rows, 0, k_width, pre, on_device(a_log), on_device(dt_bias), gates, kq, heads, key_heads, dim)
        out = torch.empty((tokens, v_width), dtype=torch.float32, device=DEVICE)
        step = packed_step(runs, slots)
        kernels.delta_rule(rows, 0, k_width, 2 * k_width, gates, kq, state, step.cu_seqlens, step.seq_slot, out, heads, key_heads, dim, vdim)
        wanted = []
        for index, pieces in enumerate(new):
            history[index] = [torch.cat([old, piece]) for old, piece in zip(history[index], pieces)]
            wanted.append(plain_delta_heads(*history[index], a_log, dt_bias, heads, key_heads, dim, vdim)[-pieces[0].shape[0] :])
        assert relative_error(out.cpu(), torch.cat(wanted)) < 2e-5
    assert not torch.equal(state[[2, 4]], torch.zeros_like(state[[2, 4]]))          # other sequences' states were left alone


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("channels, states", [(50, 1), (30, 5), (80, 8), (64, 16), (70, 32), (33, 64), (20, 128), (37, 6)])
def test_the_selective_scan_carries_its_state_from_step_to_step(dtype, channels, states):
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(channels + states)
    slots = [2, 4, 0]
    a_log = torch.log(1.0 + torch.arange(states, dtype=torch.float64)).repeat(channels, 1) + 0.2 * torch.randn(channels, states, dtype=torch.float64)
    skip = torch.randn(channels, dtype=torch.float64)
    state = torch.randn(6, channels * states, device=DEVICE)
    state[slots] = 0.0
    carried = [torch.zeros(channels, states, dtype=torch.float64) for _ in slots]
    for runs in STEPS:
        tokens = sum(runs)
        x, z = (torch.randn(tokens, channels).to(TORCH[dtype]).double() for _ in range(2))
        pre, bc = torch.randn(tokens, channels).double() - 2.0, torch.randn(tokens, 2 * states).double()
        both = on_device(torch.cat([x, z], dim=1), TORCH[dtype])
        out = torch.empty((tokens, channels), dtype=TORCH[dtype], device=DEVICE)
        step = packed_step(runs, slots)
        kernels.selective_scan(both[:, :channels], both[:, channels:], on_device(pre), on_device(bc), on_device(a_log), on_device(skip), state,
                               step.cu_seqlens, step.seq_slot, out)
        wanted, token = torch.zeros(tokens, channels, dtype=torch.float64), 0
        for index, count in enumerate(runs):
            for _ in range(count):
                size = plain.softplus(pre[token])
                carried[index] = torch.exp(size.view(-1, 1) * -torch.exp(a_log)) * carried[index] + (size * x[token]).view(-1, 1) * bc[token, :states].view(1, -1)
                wanted[token] = (carried[index] @ bc[token, states:] + skip * x[token]) * plain.silu(z[token])
                token += 1
        assert relative_error(out.float().cpu(), wanted) < (2e-5 if dtype == "float32" else 8e-3)
    assert relative_error(state[slots].cpu(), torch.stack(carried).reshape(3, -1)) < 2e-5


def attention_pages(mixer, pages, dtype, fill):
    """Pages for one layer in the layout that the sizes choose: keys and values of ordinary heads where both are 64 or 128 wide, else
    one row per position."""
    kv_heads, dim, vdim = mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    if dim == vdim and dim in (64, 128):
        return tuple(torch.full((pages, kv_heads, 64, dim), fill, dtype=TORCH[dtype], device=DEVICE) for _ in range(2))
    return torch.full((pages, 64, kv_heads * (dim + vdim)), fill, dtype=TORCH[dtype], device=DEVICE)


def run_masked_attention(h, W, mixer, eps, dtype, positions, page_of, cache, out_scale=1.0, staged=None):
    """`h` [tokens, width] of one sequence through the stacked projection in 64-bit, then the library's kernels over a paged cache
    whose pages are `page_of[position // 64]`, in the layout of `cache` (see `attention_pages`): the mixer's own two kernels, or, for
    a run of new tokens in bfloat16 over pages of ordinary heads, the tensor-core kernel behind the first of them."""
    from tau_rs_b200.csrc import kernels

    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    projected = on_device(h.double() @ torch.cat([W["m.q"], W["m.k"], W["m.v"]]).double().T, TORCH[dtype])
    tokens, rotary = h.shape[0], mixer["rot"]["dims"]
    frequency, magnitude = plain.scaled_frequencies(mixer["rot"]) if rotary else (None, 1.0)
    frequency = None if frequency is None else torch.tensor(frequency, dtype=torch.float64).float().to(DEVICE)
    step = SimpleNamespace(positions=as_ints(positions), token_seq=torch.zeros(tokens, dtype=torch.int32, device=DEVICE), n_seqs=1, all_single=tokens == 1,
                           cu_seqlens=as_ints([0, tokens]), seq_start=as_ints([positions[0]]))
    pages = as_ints([page_of])
    keys, values = cache if isinstance(cache, tuple) else (cache, None)
    queries = torch.empty((tokens, heads, dim), dtype=TORCH[dtype], device=DEVICE)
    out = torch.zeros((tokens, heads * vdim + 8), dtype=TORCH[dtype], device=DEVICE)
    kernels.masked_prepare(projected, on_device(W["m.q.norm"]), on_device(W["m.k.norm"]), eps, frequency, rotary, magnitude, queries, keys, step.positions,
                           step.token_seq, pages, heads, kv_heads, dim, vdim, True, values)
    if values is not None and dtype == "bfloat16" and tokens > 1 and not staged:
        kernels.attention_prefill_tc(queries.view(tokens, -1), keys, values, out[:, : heads * vdim], step.cu_seqlens, step.seq_start, pages, heads, kv_heads, dim,
                                     mixer["scale"], 0, mixer["mask"]["size"], True, out_scale)
        assert kernels.attention_prefill_tc_status(dim) == 0
    else:
        kernels.masked_attention(queries, keys, out[:, : heads * vdim], step, pages, kv_heads, vdim, mixer["scale"], 0, mixer["mask"]["size"], True, out_scale, values,
                                 staged=tokens == 1 if staged is None else staged)      # single tokens take the staged kernel, as in the library
    assert float(out[:, heads * vdim :].float().abs().max()) == 0.0
    return out[:, : heads * vdim].float().cpu()


def attention_weights(heads, kv_heads, dim, vdim, width):
    return {"m.q": torch.randn(heads * dim, width) / 7, "m.k": torch.randn(kv_heads * dim, width) / 7, "m.v": torch.randn(kv_heads * vdim, width) / 7,
            "m.o": torch.eye(heads * vdim), "m.q.norm": 1 + 0.2 * torch.randn(heads * dim), "m.k.norm": 1 + 0.2 * torch.randn(kv_heads * dim)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, chunk, rot_dims, scaling",
                         [(4, 2, 16, 24, 37, 8, "default"), (1, 1, 12, 150, 1, 6, "default"), (9, 3, 10, 6, 64, 10, None), (2, 1, 24, 40, 1000, 0, None),
                          (4, 2, 64, 64, 128, 64, "default"), (2, 1, 64, 128, 100, 32, pm.yarn(2.0, 20, 3.0, 1.5)), (3, 3, 48, 16, 63, 48, "default"),
                          (8, 1, 32, 64, 65, 2, None), (2, 2, 128, 128, 70, 128, "default"), (1, 1, 16, 320, 40, 4, None)])
def test_chunked_attention_kernels_over_scattered_pages(dtype, heads, kv_heads, dim, vdim, chunk, rot_dims, scaling):
    """A prompt of 150 tokens, then 60 single tokens, over pages 6, 1, 4, 0 of a pool; against the plain branch with an identity as
    its output projection.  Chunks shorter than, as long as and longer than a page, and ones that no page border divides."""
    torch.manual_seed(heads * 100 + dim)
    width, eps, total = 48, 1e-5, 210
    mixer = pm.softmax_side(heads, kv_heads, dim, vdim, chunk, rot_dims, base=300.0, scaling=scaling)
    W = attention_weights(heads, kv_heads, dim, vdim, width)
    h = torch.randn(total, width)
    wanted = plain.softmax_branch(h.double(), {name: value.double() for name, value in W.items()}, "m", mixer, eps)
    rows = attention_pages(mixer, 8, dtype, float("nan"))
    page_of = [6, 1, 4, 0]
    found = [run_masked_attention(h[:150], W, mixer, eps, dtype, list(range(150)), page_of, rows)]
    for position in range(150, 170):
        found.append(run_masked_attention(h[position : position + 1], W, mixer, eps, dtype, [position], page_of, rows))
    found.append(run_masked_attention(h[170:173], W, mixer, eps, dtype, [170, 171, 172], page_of, rows))          # a short run behind a cached prefix
    for position in range(173, total):
        found.append(run_masked_attention(h[position : position + 1], W, mixer, eps, dtype, [position], page_of, rows))
    assert relative_error(torch.cat(found), wanted) < (2e-5 if dtype == "float32" else 3e-2)
    for pool in rows if isinstance(rows, tuple) else (rows,):
        assert torch.isnan(pool[[2, 3, 5, 7]].float()).all()          # nothing was written outside the sequence's pages
    scaled = run_masked_attention(h[:150], W, mixer, eps, dtype, list(range(150)), page_of, rows, out_scale=-0.6)
    assert relative_error(scaled, -0.6 * wanted[:150]) < (2e-5 if dtype == "float32" else 3e-2)
    # the kernel of single tokens on every position of the sequence at once: tiles of 32 keys, whole and ragged, from a chunk's first key on
    tiled = run_masked_attention(h, W, mixer, eps, dtype, list(range(total)), page_of, rows, out_scale=0.5, staged=True)
    assert relative_error(tiled, 0.5 * wanted) < (2e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk, dim", [(33, 16), (64, 16), (96, 16), (33, 64), (64, 64), (96, 64), (130, 64)])      # one row per position; ordinary heads
def test_one_key_that_stands_out_is_seen_inside_the_chunk_and_not_before_it(dtype, chunk, dim):
    """Queries that point exactly along one earlier key: the first position of their own chunk for some, the last position of the
    chunk before for others (also across a page border).  A score of 64 against a spread of a few makes that key the whole softmax if
    it is seen; a chunk that is one position off changes the result altogether."""
    torch.manual_seed(9)
    heads, kv_heads, vdim, eps, total = 2, 1, 24 if dim == 16 else dim, 1e-5, 260
    width = heads * dim
    mixer = pm.softmax_side(heads, kv_heads, dim, vdim, chunk, 0, scale=64.0 / dim, scaling=None)
    # The input is the query itself: W_q is the identity, W_k picks the first head's part; unit weights, and rows of equal length so
    # that the norm over the whole projection is the same factor everywhere.
    W = {"m.q": torch.eye(heads * dim, width), "m.k": torch.zeros(kv_heads * dim, width), "m.v": torch.randn(kv_heads * vdim, width) / 5,
         "m.o": torch.eye(heads * vdim), "m.q.norm": torch.full((heads * dim,), 2.0 ** 0.5), "m.k.norm": torch.ones(kv_heads * dim)}
    W["m.k"][:, :dim] = torch.eye(dim)
    h = torch.randn(total, width).to(torch.bfloat16).float()
    inside, outside = [], []
    for index in range(1, total // chunk + 1):
        first = index * chunk
        for query, key in ((first + 7, first), (first + chunk - 1, first), (first + 1, first)):
            if query < total and query not in inside:
                h[query, :dim] = h[key, :dim]
                inside.append(query)
        for query, key in ((first + 5, first - 1), (first + 2, first - 1)):
            if query < total and query not in inside:
                h[query, :dim] = h[key, :dim]
                outside.append(query)
    weights = {name: value.double() for name, value in W.items()}
    wanted = plain.softmax_branch(h.double(), weights, "m", mixer, eps)
    page_of = [2, 0, 3, 1, 4]
    rows = attention_pages(mixer, 5, dtype, 0.0)
    whole = run_masked_attention(h, W, mixer, eps, dtype, list(range(total)), page_of, rows)
    # bfloat16 rounds queries and keys: a score of 64 moves by a quarter, its weight with it; a lost or added key moves the result by 0.3 or more
    limit = 2e-5 if dtype == "float32" else 8e-2
    assert relative_error(whole, wanted) < limit
    rows = attention_pages(mixer, 5, dtype, 0.0)
    singly = [run_masked_attention(h[:30], W, mixer, eps, dtype, list(range(30)), page_of, rows)]
    singly += [run_masked_attention(h[p : p + 1], W, mixer, eps, dtype, [p], page_of, rows) for p in range(30, total)]
    assert relative_error(torch.cat(singly), wanted) < limit
    rows = attention_pages(mixer, 5, dtype, 0.0)                                   # portions that begin inside a chunk and end in the next
    portions = [run_masked_attention(h[b : b + 52], W, mixer, eps, dtype, list(range(b, b + 52)), page_of, rows) for b in range(0, total, 52)]
    assert relative_error(torch.cat(portions), wanted) < limit
    # The test would see a chunk that is one off, either way: the plain statement itself moves by far more than the tolerance.
    for other in (chunk + 1, chunk - 1):
        moved = plain.softmax_branch(h.double(), weights, "m", {**mixer, "mask": {"size": other}}, eps)
        assert relative_error(moved[inside + outside], wanted[inside + outside]) > 0.3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [8, 64])
def test_the_added_one_in_the_denominator_takes_the_weight_that_no_key_earns(dtype, dim):
    """Every score far below zero: the result is nearly nothing, where a softmax over the keys alone would return their mean.  And
    one key alone with score 0 gets half of the weight."""
    torch.manual_seed(4)
    heads, kv_heads, vdim, eps, total = 2, 2, dim, 1e-5, 70
    width = heads * dim
    mixer = pm.softmax_side(heads, kv_heads, dim, vdim, 1000, 0, scale=8.0 / dim, scaling=None)
    W = {"m.q": torch.eye(width), "m.k": -torch.eye(width), "m.v": torch.randn(kv_heads * vdim, width), "m.o": torch.eye(heads * vdim),
         "m.q.norm": torch.full((width,), 4.0), "m.k.norm": torch.full((width,), 4.0)}
    h = (1.0 + 0.1 * torch.randn(total, width)).to(torch.bfloat16).float()          # q . k is about -16 * 8 for every pair
    h[0] = 0.0                                                                       # the first token scores 0 against itself
    h[0, 0] = 1e-6                                                                   # not all zero, yet far below the norm's eps
    wanted = plain.softmax_branch(h.double(), {name: value.double() for name, value in W.items()}, "m", mixer, eps)
    rows = attention_pages(mixer, 2, dtype, 0.0)
    found = run_masked_attention(h, W, mixer, eps, dtype, list(range(total)), [1, 0], rows)
    values = h.double() @ W["m.v"].double().T
    largest = float(values.abs().max())
    assert float(wanted[1:].abs().max()) < 1e-4 * largest                          # the statement itself: next to nothing is returned
    assert float((found.double() - wanted).abs().max()) < (1e-6 if dtype == "float32" else 1e-4) * largest
    assert relative_error(found[:1], wanted[:1]) < (2e-5 if dtype == "float32" else 2e-2)
    assert relative_error(found[0], 0.5 * values[0]) < 2e-2


@pytest.mark.parametrize("experts, top, width, ff, tokens, dtype", [(6, 2, 40, 24, 50, "float32"), (1, 1, 40, 24, 50, "float32"), (5, 5, 40, 24, 50, "float32"),
                                                                    (40, 3, 40, 24, 50, "float32"), (8, 2, 256, 64, 700, "bfloat16"), (8, 2, 256, 64, 700, "float32")])
def test_sigmoid_scores_weigh_the_chosen_experts_inputs(experts, top, width, ff, tokens, dtype):
    """The routed experts part with its weights on the inputs, against the plain routed feed-forward (SiLU, no renormalising); a few
    tokens, and enough of them for the grouped products that a long run of new tokens takes."""
    from tau_rs_b200.config.specs import RoutedExpertsSpec
    from tau_rs_b200.parts.registry import build

    torch.manual_seed(experts)
    W = {"m.router": torch.randn(experts, width) / 3}
    for expert in range(experts):
        W.update({f"m.e{expert}.gate": torch.randn(ff, width) / 4, f"m.e{expert}.up": torch.randn(ff, width) / 4, f"m.e{expert}.down": torch.randn(width, ff) / 4})
    W = {name: value.to(torch.bfloat16).float() for name, value in W.items()}
    spec = RoutedExpertsSpec(hidden=width, intermediate=ff, experts=experts, top=top, score="sigmoid", correction=False, renormalize=False, shared=None,
                             shared_gate=False, weigh="input")
    part = build("feed_forward", spec, prefix="m", dtype=TORCH[dtype], device=torch.device(DEVICE))
    for name, tensor_spec in part.tensor_specs().items():
        assert tuple(W[name].shape) == tuple(tensor_spec.shape), name
        part.assign(name, on_device(W[name], torch.float32 if name == "m.router" else TORCH[dtype]))
    part.finalize_weights()
    h = torch.randn(tokens, width).to(torch.bfloat16).float()
    found = part.forward(on_device(h, TORCH[dtype]), SimpleNamespace(all_single=False)).float().cpu()
    wanted = plain.routed_feed_forward(h.double(), {name: value.double() for name, value in W.items()}, "m", {"router": {"experts": experts, "top": top}})
    if dtype == "float32":
        assert relative_error(found, wanted) < 2e-5
    else:
        rows = (found.double() - wanted).abs().amax(dim=-1) / wanted.abs().max()
        assert float(rows.median()) < 1e-2 and float(torch.quantile(rows, 0.95)) < 3e-2


# ---- whole models: cuttings, batches, reuse --------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_whole_prompts_single_tokens_and_the_first_positions(models, name, dtype):
    engine, cfg, values = engine_of(models, name, dtype)
    tokens = tokens_for(cfg, 200, 21)
    wanted = plain_logits(cfg, values, tokens)
    whole = run_whole(engine, tokens)
    assert close(whole, wanted, dtype)
    assert close(whole[:4], wanted[:4], dtype)               # the first tokens: zeros before the convolutions, empty states, one key
    assert close(run_whole(engine, tokens[:1]), wanted[:1], dtype)
    stepwise = run_tail_stepwise(engine, tokens, 199)                              # every token but the first alone, through the graphs
    assert close(stepwise, wanted[1:], dtype)
    if dtype == "float32":
        assert relative_error(stepwise, whole[1:]) < 1e-5


def test_the_residual_stream_after_every_layer(models):
    """Layer by layer in 32-bit: the stream that the model hands from block to block against the plain statement's."""
    folder, cfg, values = models["mixed"]
    tokens = tokens_for(cfg, 90, 26)
    _, layers = plain.forward(tokens, {name: value.double() for name, value in values.items()}, cfg, return_layers=True)
    model = load_model(folder, "float32", "gpu")
    engine = Engine(model, 256)
    kept = []
    for block in model.blocks:
        original = block.forward

        def recording(hidden, *args, _original=original, **kwargs):
            result = _original(hidden, *args, **kwargs)
            kept.append(result[0].float().cpu().clone())          # (stream, pending branch)
            return result

        block.forward = recording
    run_whole(engine, tokens)
    assert len(kept) == len(cfg["layers"])
    for index, (found, wanted) in enumerate(zip(kept, layers)):
        assert relative_error(found, wanted) < 2e-5, index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "long_memory", "heady"])
def test_portions_down_to_two_tokens_and_page_borders(models, name, dtype):
    engine, cfg, values = engine_of(models, name, dtype)
    tokens = tokens_for(cfg, 330, 22)
    wanted = plain_logits(cfg, values, tokens)
    slot = engine.open_sequence()
    found, position = [], 0
    for count in [2, 2, 3, 56, 1, 1, 62, 2, 64, 1, 63, 2, 5, 64, 2]:               # runs that end at, before and behind positions 63/64, 127/128, ...
        piece = tokens[position : position + count]
        found.append(engine.step([StepEntry(slot, piece, list(range(count)))]).float().cpu().clone())
        position += count
    assert position == 330
    engine.close_sequence(slot)
    assert close(torch.cat(found), wanted, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["peaky", "edgy", "heady"])
def test_a_sharp_softmax_loses_no_key_far_back_at_a_page_border_or_at_a_chunk_edge(models, name, dtype):
    engine, cfg, values = engine_of(models, name, dtype)
    tokens = tokens_for(cfg, 400, 23)
    wanted = plain_logits(cfg, values, tokens)
    assert close(run_whole(engine, tokens), wanted, dtype)
    tail = run_tail_stepwise(engine, tokens, 150)                                  # decoded queries cross page borders and chunk edges
    assert close(tail, wanted[-150:], dtype)
    slot = engine.open_sequence()                                                  # portions whose chunks reach into earlier portions
    found = [engine.step([StepEntry(slot, tokens[begin : begin + 50], list(range(50)))]).float().cpu().clone() for begin in range(0, 400, 50)]
    engine.close_sequence(slot)
    assert close(torch.cat(found), wanted, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "edgy", "heady"])
def test_unequal_batches_against_each_request_alone(models, name, dtype):
    engine, cfg, values = engine_of(models, name, dtype, 2048)
    lengths, prompts = [90, 31, 140, 5, 66], [70, 1, 129, 3, 64]
    requests = [tokens_for(cfg, length, 30 + index) for index, length in enumerate(lengths)]
    together = run_batched(engine, requests, prompts)
    for request, prompt, rows in zip(requests, prompts, together):
        wanted = plain_logits(cfg, values, request)[prompt - 1 :]
        assert close(rows, wanted, dtype)
    engine.cache.check()
    assert engine.cache.slots.in_use == 0


def test_slots_pages_states_and_tails_that_are_used_again_start_clean(models):
    """A cache of three pages and as many slots: every request takes a slot whose states and convolution tails another left behind
    and pages that another wrote."""
    engine, cfg, values = engine_of(models, "mixed", "float32", 64 * 3)
    for round_number in range(4):
        requests = [tokens_for(cfg, length, 40 + 3 * round_number + index) for index, length in enumerate([60 + round_number, 40, 17])]
        together = run_batched(engine, requests, [len(request) - 6 for request in requests])
        for request, rows in zip(requests, together):
            assert relative_error(rows, plain_logits(cfg, values, request)[len(request) - 7 :]) < TOLERANCE["float32"]
        engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_sequence_in_a_cache_of_four_pages(models, dtype):
    """600 tokens through a cache that holds 256 positions: every attention has a chunk, so pages that lie before the current chunk are
    given back and taken again; in runs and single tokens against the plain statement of the whole sequence."""
    engine, cfg, values = engine_of(models, "edgy", dtype, 64 * 4)
    tokens = tokens_for(cfg, 600, 25)
    wanted = plain_logits(cfg, values, tokens)
    slot = engine.open_sequence()
    found, position = [], 0
    for count in [50, 1, 1, 64, 30, 1, 1, 1, 50, 50, 50, 64, 1, 50, 50, 50, 36] + [1] * 50:
        piece = tokens[position : position + count]
        found.append(engine.step([StepEntry(slot, piece, list(range(len(piece))))]).float().cpu().clone())
        position += len(piece)
        engine.cache.check()
        assert all(len(group.held[slot]) <= 3 for group in engine.cache.kv.values())
    assert position == 600
    engine.close_sequence(slot)
    assert close(torch.cat(found), wanted, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_states_that_forget_slowly_over_long_decoding(models, dtype):
    """Decays close to one: a state that was lost, restarted or carried by the wrong sequence shows hundreds of tokens later."""
    engine, cfg, values = engine_of(models, "long_memory", dtype)
    tokens = tokens_for(cfg, 420, 24)
    wanted = plain_logits(cfg, values, tokens)
    assert close(run_tail_stepwise(engine, tokens, 400), wanted[-400:], dtype)
    shortened = plain_logits(cfg, values, tokens[100:])                            # the test would see a state that began later
    assert relative_error(shortened[-50:], wanted[-50:]) > 1e-3


def test_long_decoding_in_bfloat16_stays_with_the_plain_statement(models):
    engine, cfg, values = engine_of(models, "mixed", "bfloat16")
    tokens = tokens_for(cfg, 420, 24)
    wanted = plain_logits(cfg, values, tokens)
    assert close(run_tail_stepwise(engine, tokens, 400), wanted[-400:], "bfloat16")


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_greedy_generation_through_the_library_entry_point(models, name):
    folder, cfg, values = models[name]
    prompts = [tokens_for(cfg, length, 60 + index) for index, length in enumerate([9, 30, 2])]
    output = generate(folder, prompts, max_new_tokens=12, dtype="float32", stop_tokens=[])
    for prompt, result in zip(prompts, output):
        tokens = list(prompt)
        for _ in range(12):
            logits = plain_logits(cfg, values, tokens)[-1]
            best, second = torch.topk(logits, 2).values
            if float(best - second) < 1e-3 * float(logits.abs().max()):
                break                                                                # a close call proves nothing either way
            tokens.append(int(torch.argmax(logits)))
        made = len(tokens) - len(prompt)
        assert list(result.tokens[:made]) == tokens[len(prompt) :] and made >= 1


def test_trace_replay_of_a_pegurax_folder(models, tmp_path):
    folder, cfg, values = models["odd"]
    first, second = tokens_for(cfg, 70, 70), tokens_for(cfg, 33, 71)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": first[:66], "want": [0, 65]}, {"id": "b", "tokens": second[:30], "want": [29]}], "end": []}]
    for index in range(3):
        steps.append({"step": index + 1, "entries": [{"id": "a", "tokens": [first[66 + index]], "want": [0]}, {"id": "b", "tokens": [second[30 + index]], "want": [0]}],
                      "end": ["b"] if index == 2 else []})
    steps.append({"step": 4, "entries": [{"id": "a", "tokens": [first[69]], "want": []}], "end": ["a"]})
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "256"],
                          input="\n".join(json.dumps(step) for step in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.split("\n") if line.startswith("done")] == [f"done {index}" for index in range(5)]
    wanted_a, wanted_b = plain_logits(cfg, values, first), plain_logits(cfg, values, second)
    rows = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, cfg["vocab"])
    assert relative_error(torch.from_numpy(rows), torch.stack([wanted_a[0], wanted_a[65], wanted_b[29]])) < TOLERANCE["float32"]
    rows = np.fromfile(out / "3.f32", dtype="<f4").reshape(2, cfg["vocab"])
    assert relative_error(torch.from_numpy(rows), torch.stack([wanted_a[68], wanted_b[32]])) < TOLERANCE["float32"]
    assert not (out / "4.f32").exists()


def test_the_command_line_on_a_pegurax_folder(models, tmp_path):
    """`bin/tau` on a Pegurax folder: greedy tokens in 32-bit equal those of `generate()`, with graphs and without, in chunks of
    prompt tokens; bfloat16 runs from the same folder; random weights are written for a Pegurax config.json and read back."""
    folder, cfg, values = models["mixed"]
    prompts = [tokens_for(cfg, 40, 80), tokens_for(cfg, 7, 81)]
    wanted = [list(result.tokens) for result in generate(folder, prompts, max_new_tokens=8, dtype="float32", stop_tokens=[])]

    def run(arguments):
        done = subprocess.run([os.path.join(ROOT, "bin", "tau")] + arguments, capture_output=True, text=True, timeout=900)
        assert done.returncode == 0, done.stderr[-2000:]
        return [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]

    base = ["--model", folder, "--max-tokens", "8", "--stop-ids", ""]
    for prompt in prompts:
        base += ["--prompt-ids", ",".join(str(token) for token in prompt)]
    records = run(base + ["--dtype", "f32"])
    assert [record["tokens"] for record in records if "tokens" in record] == wanted
    records = run(base + ["--dtype", "f32", "--cuda-graph", "none", "--prefill-chunk-size", "16"])
    assert [record["tokens"] for record in records if "tokens" in record] == wanted
    records = run(base + ["--dtype", "bf16"])
    assert all(len(record["tokens"]) == 8 for record in records if "tokens" in record)
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(pm.PEAKY))
    drawn = str(tmp_path / "drawn")
    records = run(["--random-weights", str(config_path), "--model", drawn, "--seed", "4", "--max-tokens", "5", "--stop-ids", "", "--prompt-ids", "1,2,3"])
    assert [len(record["tokens"]) for record in records if "tokens" in record] == [5]
