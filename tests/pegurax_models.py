"""Small Pegurax configurations and weights for the tests, made here from the config alone (names, shapes and scales are written
out by hand; nothing is taken from the library's own list of tensors)."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from tau_rs_b200.weights.safetensors_io import write_safetensors


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=40):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def yarn(factor=4.0, original=64, fast=16.0, slow=2.0):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def softmax_side(heads=4, kv_heads=2, dim=16, vdim=24, chunk=37, rot_dims=8, base=5000.0, scale=None, scaling="default"):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = yarn() if scaling == "default" else scaling
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale, "mask": {"size": chunk}, "rot": rot}


def delta_side(heads=4, kv_heads=2, dim=16, vdim=24, conv=4):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(left=None, right=None, left_scale=0.7, right_scale=1.3, mlp="default"):
    return {"type": "parallel", "mixer": {"left": left or softmax_side(), "right": right or delta_side(), "left_scale": left_scale, "right_scale": right_scale},
            "mlp": dense() if mlp == "default" else mlp}


def mamba(inner=80, state=8, dt_rank=6, conv=3, mlp="default"):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": dense() if mlp == "default" else mlp}


def config(layers, width=96, vocab=211, eps=1e-5, embedding_scale=0.75) -> dict:
    return {"architecture": "Pegurax", "embedding": {"scale": embedding_scale}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


# Both mixers, both feed-forwards and none; chunks shorter and longer than a page; rotations narrower than and as wide as a head,
# scaled and plain; two mixers of a kind with different sizes; a scan behind a scan.
MIXED = config([parallel(),
                mamba(mlp=moe()),
                parallel(softmax_side(heads=6, kv_heads=3, dim=8, vdim=40, chunk=70, rot_dims=8, scaling=None), delta_side(heads=6, kv_heads=2, dim=24, vdim=8, conv=2),
                         left_scale=1.2, right_scale=0.4, mlp=None),
                mamba(inner=48, state=16, dt_rank=3, conv=4, mlp=moe(experts=5, top=3, ff=24)),
                mamba(inner=64, state=4, dt_rank=8, conv=2, mlp=None)])
# Sizes that happen to be 1 or equal elsewhere, and nothing a multiple of 8: one head, a chunk of one position, one tap (no tail), one
# expert of one, all experts chosen, values wider than a warp's pass, key heads as many as heads, one state, a step size from one
# number, scales of one and below zero, an embedding that is not scaled.
ODD = config([parallel(softmax_side(heads=1, kv_heads=1, dim=12, vdim=150, chunk=1, rot_dims=6), delta_side(heads=1, kv_heads=1, dim=20, vdim=70, conv=1),
                       left_scale=1.0, right_scale=-0.5, mlp=moe(experts=1, top=1, ff=20)),
              mamba(inner=50, state=1, dt_rank=1, conv=1, mlp=moe(experts=4, top=4, ff=12)),
              parallel(softmax_side(heads=9, kv_heads=3, dim=10, vdim=6, chunk=5, rot_dims=10, scaling=yarn(2.0, 20, 3.0, 1.5)),
                       delta_side(heads=3, kv_heads=3, dim=6, vdim=34, conv=7), left_scale=0.3, right_scale=1.0, mlp=dense(ff=30)),
              mamba(inner=30, state=5, dt_rank=11, conv=5, mlp=dense(ff=14)),
              parallel(softmax_side(heads=2, kv_heads=1, dim=20, vdim=34, chunk=1000, rot_dims=2, scaling=None), delta_side(heads=2, kv_heads=1, dim=100, vdim=10, conv=2),
                       mlp=None)], width=100, vocab=77, eps=1e-6, embedding_scale=1.0)
# Attention with a sharp softmax, so that single keys carry a query's weight: a key lost far back, at a page border or at a chunk's
# edge, or one seen beyond it, moves the logits by much more than rounding does.  The delta rule beside it is kept quiet.
PEAKY = config([parallel(softmax_side(heads=3, kv_heads=1, dim=16, vdim=24, chunk=300, rot_dims=16, scale=3.0), delta_side(heads=2, kv_heads=1, dim=8, vdim=8, conv=3),
                         left_scale=1.0, right_scale=0.05, mlp=None)], width=64, vocab=97)
EDGY = config([parallel(softmax_side(heads=4, kv_heads=2, dim=16, vdim=16, chunk=33, rot_dims=4, scale=4.0), delta_side(heads=2, kv_heads=1, dim=8, vdim=8, conv=4),
                        left_scale=1.0, right_scale=0.05, mlp=None),
               parallel(softmax_side(heads=2, kv_heads=1, dim=16, vdim=32, chunk=64, rot_dims=16, scale=4.0, scaling=None), delta_side(heads=2, kv_heads=1, dim=8, vdim=8, conv=2),
                        left_scale=1.0, right_scale=0.05, mlp=None)], width=64, vocab=97)
# The same with keys and values as wide as ordinary heads (64 and 128), which the library keeps in another cache layout and, for runs
# of tokens in bfloat16, hands to another attention kernel; chunks that no page border divides.
HEADY = config([parallel(softmax_side(heads=2, kv_heads=1, dim=64, vdim=64, chunk=96, rot_dims=32, scale=2.0), delta_side(heads=2, kv_heads=1, dim=8, vdim=8, conv=4),
                         left_scale=1.0, right_scale=0.05, mlp=None),
                parallel(softmax_side(heads=2, kv_heads=2, dim=128, vdim=128, chunk=50, rot_dims=128, scale=1.4, scaling=None), delta_side(heads=2, kv_heads=1, dim=8, vdim=8, conv=2),
                         left_scale=1.0, right_scale=0.05, mlp=None)], width=64, vocab=97)
# Recurrences only slowly forgetting, so that a state lost or restarted shows hundreds of tokens later.
LONG_MEMORY = config([parallel(softmax_side(heads=2, kv_heads=2, dim=8, vdim=8, chunk=16), delta_side(heads=4, kv_heads=1, dim=32, vdim=16, conv=4),
                               left_scale=0.1, right_scale=1.5, mlp=None),
                      mamba(inner=64, state=32, dt_rank=4, conv=4, mlp=None)], width=64, vocab=53)


def weights(cfg: dict, seed: int, slow_decay: bool = False) -> Dict[str, torch.Tensor]:
    """Random weights of the scales that keep every branch alive, every value one that bfloat16 holds.  `slow_decay`: the delta
    rule's and the scan's decays stay close to one."""
    generator = torch.Generator().manual_seed(seed)
    width = cfg["width"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, columns, gain=1.0):
        out[name] = torch.randn(rows, columns, generator=generator) * gain / columns ** 0.5

    def vector(name, count, mean, spread):
        out[name] = mean + spread * torch.randn(count, generator=generator)

    def feed_forward(prefix, ff):
        matrix(f"{prefix}.gate", ff, width, 1.5)
        matrix(f"{prefix}.up", ff, width, 1.5)
        matrix(f"{prefix}.down", width, ff)

    out["embed"] = torch.randn(cfg["vocab"], width, generator=generator)
    vector("final.norm", width, 0.2, 0.05)
    for index, layer in enumerate(cfg["layers"]):
        p, mixer, mlp = f"l{index}", layer["mixer"], layer["mlp"]
        vector(f"{p}.norm1", width, 0.7, 0.2)
        vector(f"{p}.norm1b", width, 1.0, 0.3)
        vector(f"{p}.ls1", width, 0.5, 0.2)
        if layer["type"] == "parallel":
            left, right = mixer["left"], mixer["right"]
            heads, kv_heads, dim, vdim = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
            matrix(f"{p}.mix.left.q", heads * dim, width)
            matrix(f"{p}.mix.left.k", kv_heads * dim, width)
            matrix(f"{p}.mix.left.v", kv_heads * vdim, width)
            matrix(f"{p}.mix.left.o", width, heads * vdim)
            vector(f"{p}.mix.left.q.norm", heads * dim, 1.0, 0.2)
            vector(f"{p}.mix.left.k.norm", kv_heads * dim, 1.0, 0.2)
            heads, kv_heads, dim, vdim, taps = right["heads"], right["kv_heads"], right["dim"], right["vdim"], right["conv"]
            for name, rows in (("q", kv_heads * dim), ("k", kv_heads * dim), ("v", heads * vdim)):
                matrix(f"{p}.mix.right.{name}", rows, width, 2.0)
                out[f"{p}.mix.right.{name}.conv"] = 0.5 * torch.randn(rows, taps, generator=generator) + (0.5 if taps == 1 else 0.0)
            matrix(f"{p}.mix.right.g", heads * vdim, width, 2.0)
            matrix(f"{p}.mix.right.o", width, heads * vdim)
            matrix(f"{p}.mix.right.b", heads, width, 2.0)
            matrix(f"{p}.mix.right.a", heads, width, 2.0)
            vector(f"{p}.mix.right.A_log", heads, -4.0 if slow_decay else -0.5, 0.5)
            vector(f"{p}.mix.right.dt_bias", heads, 0.0, 0.7)
            vector(f"{p}.mix.right.norm", vdim, 1.0, 0.2)
        else:
            inner, states, rank, taps = mixer["inner"], mixer["state"], mixer["dt_rank"], mixer["conv"]
            matrix(f"{p}.mix.in", 2 * inner, width, 2.0)
            out[f"{p}.mix.conv"] = 0.5 * torch.randn(inner, taps, generator=generator) + (0.5 if taps == 1 else 0.0)
            vector(f"{p}.mix.conv.b", inner, 0.0, 0.2)
            matrix(f"{p}.mix.x", rank + 2 * states, inner, 2.0)
            matrix(f"{p}.mix.dt", inner, rank, 1.0)
            vector(f"{p}.mix.dt.b", inner, -4.0 if slow_decay else -1.0, 0.7)
            out[f"{p}.mix.A_log"] = torch.log(1.0 + torch.arange(states, dtype=torch.float32)).repeat(inner, 1) + 0.2 * torch.randn(inner, states, generator=generator)
            vector(f"{p}.mix.D", inner, 1.0, 0.3)
            matrix(f"{p}.mix.o", width, inner)
        if mlp is not None:
            vector(f"{p}.norm2", width, 0.7, 0.2)
            vector(f"{p}.norm2b", width, 1.0, 0.3)
            vector(f"{p}.ls2", width, 0.5, 0.2)
            if mlp["kind"] == "dense":
                feed_forward(f"{p}.mlp", mlp["ff"])
            else:
                matrix(f"{p}.mlp.router", mlp["router"]["experts"], width, 2.0)
                for expert in range(mlp["router"]["experts"]):
                    feed_forward(f"{p}.mlp.e{expert}", mlp["expert"]["ff"])
    return {name: value.to(torch.bfloat16).float() for name, value in out.items()}


def write_model(folder: str, cfg: dict, seed: int, storage=torch.bfloat16, values=None, slow_decay: bool = False) -> Dict[str, torch.Tensor]:
    os.makedirs(folder, exist_ok=True)
    values = weights(cfg, seed, slow_decay) if values is None else values
    write_safetensors(os.path.join(folder, "model.safetensors"), ((name, value.to(storage)) for name, value in values.items()))
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(cfg, handle)
    return values
