"""Small Nugolorn configurations and weights for the tests, made here from the config alone (names, shapes and scales are written
out by hand; nothing is taken from the library's own list of tensors)."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from tau_rs_b200.weights.safetensors_io import write_safetensors


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, identity=2, top=3, ff=40):
    return {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff}}


def attention(heads=4, kv_heads=2, dim=16, vdim=24, conv=4, rot_dims=8, base=5000.0, scale=None, kv_from=None, mlp="default"):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if conv:
        mixer["conv"] = conv
    if rot_dims:
        mixer["rot"] = {"base": base, "dims": rot_dims}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": dense() if mlp == "default" else mlp}


def wkv(heads=3, dim=16, rank=6, mlp="default"):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}, "mlp": dense() if mlp == "default" else mlp}


def softmax_side(heads=4, kv_heads=2, dim=16, vdim=24, scale=None, coef=0.4, every=16):
    side = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if every:
        side["q_temp"] = {"coef": coef, "every": every}
    return side


def delta_side(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, decay_rank=5, gate_rank=7):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank, "gate_rank": gate_rank}


def parallel(left=None, right=None, mlp="default"):
    return {"type": "parallel", "mixer": {"left": left or softmax_side(), "right": right or delta_side()}, "mlp": dense() if mlp == "default" else mlp}


def config(layers, width=96, vocab=211, eps=1e-5, groups=3, residual_mult=0.6, logit_scale=0.5) -> dict:
    return {"architecture": "Nugolorn", "layers": layers, "norm": {"eps": eps, "groups": groups}, "residual_mult": residual_mult, "logit_scale": logit_scale,
            "vocab": vocab, "width": width}


# Every mixer, every feed-forward and none; a layer that reads the keys of the first and one that reads those of another; rotations
# narrower than and as wide as a head; two mixers of a kind with different sizes.
MIXED = config([attention(),
                wkv(mlp=moe()),
                parallel(),
                attention(heads=6, kv_heads=2, kv_from=0, mlp=moe(experts=4, identity=3, top=2, ff=24)),
                attention(heads=2, kv_heads=1, dim=8, vdim=40, conv=2, rot_dims=8, mlp=None),
                wkv(heads=2, dim=24, rank=3, mlp=None),
                parallel(softmax_side(heads=6, kv_heads=3, dim=8, vdim=40, every=5), delta_side(heads=6, kv_heads=2, dim=24, vdim=8, conv=2, decay_rank=3, gate_rank=2),
                         mlp=moe()),
                attention(heads=4, kv_heads=1, dim=8, vdim=40, conv=2, rot_dims=8, kv_from=4)])
# Sizes that happen to be 1 or equal elsewhere, and nothing a multiple of 8: one head, one tap (no tail) and no convolution at all, no
# rotation, values wider than a warp's pass, key heads as many as heads, one group in the norm and as many as the width allows, a
# temperature that changes at every position and none, one expert, all router outputs chosen, no identity experts and nothing but
# them beside one expert, ranks of one, factors of one and above.
ODD = config([attention(heads=1, kv_heads=1, dim=12, vdim=150, conv=1, rot_dims=6, mlp=moe(experts=1, identity=0, top=1, ff=20)),
              wkv(heads=1, dim=20, rank=1, mlp=moe(experts=3, identity=1, top=4, ff=12)),
              parallel(softmax_side(heads=1, kv_heads=1, dim=12, vdim=150, every=1), delta_side(heads=1, kv_heads=1, dim=20, vdim=70, conv=1, decay_rank=1, gate_rank=1),
                       mlp=moe(experts=1, identity=4, top=2, ff=10)),
              attention(heads=9, kv_heads=3, dim=10, vdim=6, conv=0, rot_dims=0, mlp=dense(ff=30)),
              parallel(softmax_side(heads=9, kv_heads=3, dim=10, vdim=6, every=0), delta_side(heads=3, kv_heads=3, dim=6, vdim=34, conv=7), mlp=None),
              attention(heads=3, kv_heads=3, dim=10, vdim=6, conv=5, rot_dims=0, kv_from=3, mlp=None),
              wkv(heads=5, dim=6, rank=9, mlp=dense(ff=14)),
              parallel(softmax_side(heads=2, kv_heads=1, dim=20, vdim=34), delta_side(heads=2, kv_heads=1, dim=100, vdim=10, conv=2), mlp=None)],
             width=100, vocab=77, eps=1e-6, groups=1, residual_mult=1.0, logit_scale=1.0)
MANY_GROUPS = config([attention(mlp=None), wkv(mlp=None)], width=100, vocab=77, groups=50, residual_mult=1.7, logit_scale=3.0)
# Attention with sharp weights, so that single keys carry a query's result: a key lost far back or at a page border moves the logits by
# much more than rounding does.  The delta rule beside the softmax is kept quiet (its share of the mixer's result is made small).
PEAKY = config([parallel(softmax_side(heads=3, kv_heads=1, dim=16, vdim=24, scale=3.0, every=64), delta_side(heads=2, kv_heads=1, dim=8, vdim=8), mlp=None),
                attention(heads=3, kv_heads=1, dim=16, vdim=24, scale=3.0, conv=2, rot_dims=16, mlp=None)], width=64, vocab=97, groups=2)
# The same with keys and values as wide as ordinary heads (64 and 128), which the library keeps in another cache layout.
HEADY = config([parallel(softmax_side(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.5), delta_side(heads=2, kv_heads=1, dim=8, vdim=8), mlp=None),
                attention(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.25, conv=3, rot_dims=64, mlp=None),
                attention(heads=4, kv_heads=2, dim=128, vdim=128, scale=0.25, conv=3, rot_dims=64, kv_from=1, mlp=None)], width=64, vocab=97, groups=4)
# Recurrences only slowly forgetting, so that a state lost or restarted shows hundreds of tokens later.
LONG_MEMORY = config([parallel(softmax_side(heads=2, kv_heads=2, dim=8, vdim=8), delta_side(heads=4, kv_heads=1, dim=32, vdim=16, conv=4), mlp=None),
                      wkv(heads=2, dim=32, rank=4, mlp=None)], width=64, vocab=53, groups=2)
# One mechanism to a model.
ONLY = {
    "attention": config([attention(mlp=None)], width=64, vocab=61, groups=2),
    "shared_keys": config([attention(mlp=None), attention(heads=2, kv_heads=2, kv_from=0, mlp=None)], width=64, vocab=61, groups=2),
    "wkv": config([wkv(mlp=None)], width=64, vocab=61, groups=2),
    "parallel": config([parallel(mlp=None)], width=64, vocab=61, groups=2),
    "experts": config([attention(heads=1, kv_heads=1, dim=8, vdim=8, conv=0, rot_dims=0, mlp=moe(experts=6, identity=3, top=4, ff=24))], width=64, vocab=61, groups=2),
}


def weights(cfg: dict, seed: int, slow_decay: bool = False, quiet_delta: bool = False) -> Dict[str, torch.Tensor]:
    """Random weights of the scales that keep every branch alive, every value one that bfloat16 holds.  `slow_decay`: the recurrences'
    decays stay close to one.  `quiet_delta`: the delta rule's share of a parallel mixer's result is small."""
    generator = torch.Generator().manual_seed(seed)
    width = cfg["width"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, columns, gain=1.0):
        out[name] = torch.randn(rows, columns, generator=generator) * gain / columns ** 0.5

    def vector(name, count, mean, spread):
        out[name] = mean + spread * torch.randn(count, generator=generator)

    def taps(name, rows, count):
        out[name] = 0.5 * torch.randn(rows, count, generator=generator) + (0.5 if count == 1 else 0.0)

    def feed_forward(prefix, ff):
        matrix(f"{prefix}.gate", ff, width, 1.5)
        matrix(f"{prefix}.up", ff, width, 1.5)
        matrix(f"{prefix}.down", width, ff)

    out["embed"] = torch.randn(cfg["vocab"], width, generator=generator)
    matrix("head", cfg["vocab"], width, 2.0)
    vector("final.norm", width, 1.0, 0.2)
    for index, layer in enumerate(cfg["layers"]):
        p, mixer, mlp = f"l{index}", layer["mixer"], layer["mlp"]
        vector(f"{p}.norm1", width, 0.7, 0.2)
        if layer["type"] == "attention":
            heads, kv_heads, dim, vdim, count = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"], mixer.get("conv", 0)
            own = ("q", "k", "v") if mixer.get("kv_from") is None else ("q",)
            for name, rows in (("q", heads * dim), ("k", kv_heads * dim), ("v", kv_heads * vdim)):
                if name in own:
                    matrix(f"{p}.mix.{name}", rows, width, 2.0)
                    vector(f"{p}.mix.{name}.b", rows, 0.0, 0.3)
                    if count:
                        taps(f"{p}.mix.{name}.conv", rows, count)
            vector(f"{p}.mix.pb", heads, -1.0, 0.7)
            matrix(f"{p}.mix.g", heads, width, 2.0)
            matrix(f"{p}.mix.o", width, heads * vdim, 0.5)
        elif layer["type"] == "wkv":
            heads, dim, rank = mixer["heads"], mixer["dim"], mixer["decay_rank"]
            for name in ("r", "k", "v", "g", "w"):
                out[f"{p}.mix.mu.{name}"] = torch.rand(width, generator=generator)
            for name in ("r", "k", "v", "g"):
                matrix(f"{p}.mix.{name}", heads * dim, width, 1.5)
            matrix(f"{p}.mix.w1", rank, width, 1.5)
            matrix(f"{p}.mix.w2", heads * dim, rank, 1.5)
            vector(f"{p}.mix.w0", heads * dim, -5.0 if slow_decay else -1.0, 0.7)
            out[f"{p}.mix.u"] = 0.5 * torch.randn(heads, dim, generator=generator)
            vector(f"{p}.mix.norm", heads * dim, 1.0, 0.2)
            matrix(f"{p}.mix.o", width, heads * dim)
        else:
            left, right = mixer["left"], mixer["right"]
            heads, kv_heads, dim, vdim = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
            matrix(f"{p}.mix.left.q", heads * dim, width, 2.0)
            matrix(f"{p}.mix.left.k", kv_heads * dim, width, 2.0)
            matrix(f"{p}.mix.left.v", kv_heads * vdim, width, 2.0)
            matrix(f"{p}.mix.left.g", heads * vdim, width, 2.0)
            matrix(f"{p}.mix.left.o", width, heads * vdim)
            out[f"{p}.mix.left.r1"] = 0.3 * torch.rand(heads, generator=generator)
            out[f"{p}.mix.left.r2"] = 0.2 + torch.rand(heads, generator=generator)
            vector(f"{p}.mix.left.out", width, 1.0, 0.2)
            heads, kv_heads, dim, vdim, count = right["heads"], right["kv_heads"], right["dim"], right["vdim"], right["conv"]
            for name, rows in (("q", kv_heads * dim), ("k", kv_heads * dim), ("v", heads * vdim)):
                matrix(f"{p}.mix.right.{name}", rows, width, 2.0)
                taps(f"{p}.mix.right.{name}.conv", rows, count)
            matrix(f"{p}.mix.right.b", heads, width, 2.0)
            matrix(f"{p}.mix.right.a1", right["decay_rank"], width, 2.0)
            matrix(f"{p}.mix.right.a2", heads * dim, right["decay_rank"], 2.0)
            matrix(f"{p}.mix.right.g1", right["gate_rank"], width, 2.0)
            matrix(f"{p}.mix.right.g2", heads * vdim, right["gate_rank"], 2.0)
            matrix(f"{p}.mix.right.o", width, heads * vdim)
            vector(f"{p}.mix.right.A_log", heads, -4.0 if slow_decay else -0.5, 0.5)
            vector(f"{p}.mix.right.dt_bias", heads * dim, 0.0, 0.7)
            vector(f"{p}.mix.right.norm", vdim, 1.0, 0.2)
            vector(f"{p}.mix.right.out", width, 0.05 if quiet_delta else 1.0, 0.01 if quiet_delta else 0.2)
        if mlp is not None:
            if mlp["kind"] == "dense":
                feed_forward(f"{p}.mlp", mlp["ff"])
            else:
                outputs = mlp["router"]["experts"] + mlp["router"].get("identity", 0)
                matrix(f"{p}.mlp.router", outputs, width, 3.0)
                vector(f"{p}.mlp.correction", outputs, 0.0, 0.1)
                for expert in range(mlp["router"]["experts"]):
                    feed_forward(f"{p}.mlp.e{expert}", mlp["expert"]["ff"])
    return {name: value.to(torch.bfloat16).float() for name, value in out.items()}


def write_model(folder: str, cfg: dict, seed: int, storage=torch.bfloat16, values=None, slow_decay: bool = False, quiet_delta: bool = False,
                ranks_in_config: bool = True) -> Dict[str, torch.Tensor]:
    """`ranks_in_config=False` leaves the low ranks out of config.json, as a folder does whose tensors' shapes alone give them."""
    os.makedirs(folder, exist_ok=True)
    values = weights(cfg, seed, slow_decay, quiet_delta) if values is None else values
    write_safetensors(os.path.join(folder, "model.safetensors"), ((name, value.to(storage)) for name, value in values.items()))
    written = json.loads(json.dumps(cfg))
    if not ranks_in_config:
        for layer in written["layers"]:
            layer["mixer"].pop("decay_rank", None)
            for key in ("decay_rank", "gate_rank"):
                layer["mixer"].get("right", {}).pop(key, None)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(written, handle)
    return values
