"""Nugolorn stated plainly: one function per mechanism, float64, whole sequences, masks instead of caches, loops over tokens
instead of carried state.

Shares nothing with the library.  `weights` maps tensor names to float64 tensors, `config` is the dictionary that a folder's
config.json holds.  Every function takes one sequence `[tokens, ...]` whose first row is position 0.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def grouped_rms_norm(x, weight, groups, eps):
    """The row is cut into `groups` equal consecutive pieces; each is divided by its own root mean square."""
    tokens, width = x.shape
    pieces = x.reshape(tokens, groups, width // groups)
    return unit_rms(pieces, eps).reshape(tokens, width) * weight


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_convolution(x, taps_weight):
    """`out[t, c] = sum_j w[c, j] * x[t - (taps - 1) + j, c]`: the last column weighs the token itself, rows before the start are zero."""
    tokens, taps = x.shape[0], taps_weight.shape[1]
    out = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < tokens:
            out[back:] += taps_weight[:, j] * x[: tokens - back]
    return out


def rotate_halves(x, rot):
    """x [tokens, heads, dim]: element i of the first `dims` is paired with element i + dims / 2; the rest pass."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    tokens = x.shape[0]
    frequency = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = torch.arange(tokens, dtype=F)[:, None] * frequency[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def sigmoid_attention(q, k, v, scale, offset):
    """q [tokens, heads, dim], k [tokens, kv_heads, dim], v [tokens, kv_heads, vdim], offset [heads]: every visible key weighs
    sigmoid(score + offset); the weights are not normalised over the keys."""
    tokens, heads, _ = q.shape
    per = heads // k.shape[1]
    visible = torch.tril(torch.ones(tokens, tokens, dtype=torch.bool))
    out = torch.zeros(tokens, heads, v.shape[-1], dtype=F)
    for head in range(heads):
        score = q[:, head] @ k[:, head // per].T * scale + offset[head]
        weight = torch.where(visible, torch.sigmoid(score), torch.zeros((), dtype=F))
        out[:, head] = weight @ v[:, head // per]
    return out


def distance_softmax_attention(q, k, v, scale, r1, r2):
    """Softmax over the keys j <= i of `q_i . k_j * scale - r1 * ln(1 + r2 * (i - j))`, r1 and r2 one number per head."""
    tokens, heads, _ = q.shape
    per = heads // k.shape[1]
    place = torch.arange(tokens, dtype=F)
    distance = place[:, None] - place[None, :]
    visible = distance >= 0
    out = torch.zeros(tokens, heads, v.shape[-1], dtype=F)
    for head in range(heads):
        score = q[:, head] @ k[:, head // per].T * scale - r1[head] * torch.log1p(r2[head] * distance.clamp(min=0.0))
        score = torch.where(visible, score, torch.full((), -math.inf, dtype=F))
        out[:, head] = torch.softmax(score, dim=-1) @ v[:, head // per]
    return out


def conv_attention_mixer(h, weights, prefix, mixer, kept=None):
    """The `attention` mixer.  Returns (output, (keys, values)) so that a later layer can read this one's keys and values; such a
    layer passes them as `kept` and has no key or value tensors of its own."""
    tokens = h.shape[0]
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]

    def projected(name):
        result = h @ weights[f"{prefix}.{name}"].T + weights[f"{prefix}.{name}.b"]
        return causal_convolution(result, weights[f"{prefix}.{name}.conv"]) if mixer.get("conv") else result

    q = projected("q").reshape(tokens, heads, dim)
    if "rot" in mixer and mixer["rot"] is not None:
        q = rotate_halves(q, mixer["rot"])
    if kept is None:
        k = projected("k").reshape(tokens, kv_heads, dim)
        if "rot" in mixer and mixer["rot"] is not None:
            k = rotate_halves(k, mixer["rot"])
        v = projected("v").reshape(tokens, kv_heads, vdim)
    else:
        k, v = kept
    out = sigmoid_attention(q, k, v, mixer["scale"], weights[f"{prefix}.pb"])
    gate = torch.sigmoid(h @ weights[f"{prefix}.g"].T)                      # [tokens, heads]
    out = (out * gate[:, :, None]).reshape(tokens, heads * vdim)
    return out @ weights[f"{prefix}.o"].T, (k, v)


def softmax_side(h, weights, prefix, mixer):
    tokens = h.shape[0]
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    q = (h @ weights[f"{prefix}.q"].T).reshape(tokens, heads, dim)
    k = (h @ weights[f"{prefix}.k"].T).reshape(tokens, kv_heads, dim)
    v = (h @ weights[f"{prefix}.v"].T).reshape(tokens, kv_heads, vdim)
    temperature = mixer.get("q_temp")
    if temperature is not None:
        place = torch.arange(tokens, dtype=F)
        factor = 1.0 + temperature["coef"] * torch.log(torch.floor((place + 1.0) / temperature["every"]) + 1.0)
        q = q * factor[:, None, None]
    out = distance_softmax_attention(q, k, v, mixer["scale"], weights[f"{prefix}.r1"], weights[f"{prefix}.r2"])
    out = out.reshape(tokens, heads * vdim) * torch.sigmoid(h @ weights[f"{prefix}.g"].T)
    return out @ weights[f"{prefix}.o"].T


def channel_gated_delta_rule(q, k, v, beta, decay):
    """q, k [tokens, heads, dim] (already per value head), v [tokens, heads, vdim], beta [tokens, heads], decay [tokens, heads, dim]:
    a decay per key channel on the rows of the state."""
    tokens, heads, dim = q.shape
    state = torch.zeros(heads, dim, v.shape[-1], dtype=F)
    out = torch.zeros_like(v)
    for t in range(tokens):
        state = decay[t][:, :, None] * state
        update = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", state, k[t]))
        state = state + k[t][:, :, None] * update[:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    return out


def delta_side(h, weights, prefix, mixer, eps):
    tokens = h.shape[0]
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    per = heads // kv_heads

    def projected(name):
        return silu(causal_convolution(h @ weights[f"{prefix}.{name}"].T, weights[f"{prefix}.{name}.conv"]))

    q = projected("q").reshape(tokens, kv_heads, dim)
    k = projected("k").reshape(tokens, kv_heads, dim)
    v = projected("v").reshape(tokens, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(per, dim=1), k.repeat_interleave(per, dim=1)
    beta = torch.sigmoid(h @ weights[f"{prefix}.b"].T)
    step = softplus((h @ weights[f"{prefix}.a1"].T) @ weights[f"{prefix}.a2"].T + weights[f"{prefix}.dt_bias"]).reshape(tokens, heads, dim)
    decay = torch.exp(-torch.exp(weights[f"{prefix}.A_log"])[None, :, None] * step)
    read = channel_gated_delta_rule(q, k, v, beta, decay)
    gate = torch.sigmoid((h @ weights[f"{prefix}.g1"].T) @ weights[f"{prefix}.g2"].T).reshape(tokens, heads, vdim)
    out = unit_rms(read, eps) * weights[f"{prefix}.norm"] * gate
    return out.reshape(tokens, heads * vdim) @ weights[f"{prefix}.o"].T


def parallel_mixer(h, weights, prefix, mixer, eps):
    left = softmax_side(h, weights, f"{prefix}.left", mixer["left"])
    right = delta_side(h, weights, f"{prefix}.right", mixer["right"], eps)
    return 0.5 * (unit_rms(left, eps) * weights[f"{prefix}.left.out"] + unit_rms(right, eps) * weights[f"{prefix}.right.out"])


def wkv_recurrence(r, k, v, w, bonus):
    """r, k, w [tokens, heads, dim], v [tokens, heads, vdim], bonus [heads, dim]: the read-out sees the states of the tokens before
    and the token's own k v^T weighed by the bonus; the state then decays and takes k v^T unweighed."""
    tokens, heads, dim = r.shape
    state = torch.zeros(heads, dim, v.shape[-1], dtype=F)
    out = torch.zeros_like(v)
    for t in range(tokens):
        own = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state + bonus[:, :, None] * own, r[t])
        state = w[t][:, :, None] * state + own
    return out


def wkv_mixer(h, weights, prefix, mixer, eps):
    tokens = h.shape[0]
    heads, dim = mixer["heads"], mixer["dim"]
    before = torch.cat([torch.zeros(1, h.shape[1], dtype=F), h[:-1]], dim=0)

    def mixed(name):
        return h + (before - h) * weights[f"{prefix}.mu.{name}"]

    r = (mixed("r") @ weights[f"{prefix}.r"].T).reshape(tokens, heads, dim)
    k = (mixed("k") @ weights[f"{prefix}.k"].T).reshape(tokens, heads, dim)
    v = (mixed("v") @ weights[f"{prefix}.v"].T).reshape(tokens, heads, dim)
    gate = silu(mixed("g") @ weights[f"{prefix}.g"].T)
    w = torch.exp(-torch.exp(torch.tanh(mixed("w") @ weights[f"{prefix}.w1"].T) @ weights[f"{prefix}.w2"].T + weights[f"{prefix}.w0"]))
    read = wkv_recurrence(r, k, v, w.reshape(tokens, heads, dim), weights[f"{prefix}.u"])
    out = unit_rms(read, eps).reshape(tokens, heads * dim) * weights[f"{prefix}.norm"] * gate
    return out @ weights[f"{prefix}.o"].T


def gated_feed_forward(h, weights, prefix):
    return (silu(h @ weights[f"{prefix}.gate"].T) * (h @ weights[f"{prefix}.up"].T)) @ weights[f"{prefix}.down"].T


def routed_feed_forward(h, weights, prefix, mlp):
    """Softmax over all router outputs; chosen by score + correction, weighed by the score alone; the last `identity` outputs stand
    for experts that return their input."""
    router = mlp["router"]
    experts, identity, top = router["experts"], router.get("identity", 0), router["top"]
    score = torch.softmax(h @ weights[f"{prefix}.router"].T, dim=-1)
    chosen = torch.topk(score + weights[f"{prefix}.correction"], top, dim=-1).indices
    out = torch.zeros_like(h)
    for token in range(h.shape[0]):
        for e in chosen[token].tolist():
            row = h[token : token + 1]
            result = gated_feed_forward(row, weights, f"{prefix}.e{e}") if e < experts else row
            out[token] += score[token, e] * result[0]
    return out


def forward(tokens, weights, config, return_layers=False):
    """Logits [tokens, vocab] of one sequence (and, if asked, the residual stream after every layer)."""
    eps, groups, m = config["norm"]["eps"], config["norm"].get("groups", 1), config.get("residual_mult", 1.0)
    x = weights["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept, streams = {}, []
    for index, layer in enumerate(config["layers"]):
        prefix, mixer = f"l{index}", layer["mixer"]
        h = grouped_rms_norm(x, weights[f"{prefix}.norm1"], groups, eps)
        if layer["type"] == "attention":
            source = mixer.get("kv_from")
            mixed, kept[index] = conv_attention_mixer(h, weights, f"{prefix}.mix", mixer, None if source is None else kept[source])
        elif layer["type"] == "wkv":
            mixed = wkv_mixer(h, weights, f"{prefix}.mix", mixer, eps)
        elif layer["type"] == "parallel":
            mixed = parallel_mixer(h, weights, f"{prefix}.mix", mixer, eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            mixed = mixed + (gated_feed_forward(h, weights, f"{prefix}.mlp") if mlp["kind"] == "dense" else routed_feed_forward(h, weights, f"{prefix}.mlp", mlp))
        x = x + m * mixed
        streams.append(x)
    logits = grouped_rms_norm(x, weights["final.norm"], groups, eps) @ weights["head"].T * config.get("logit_scale", 1.0)
    return (logits, torch.stack(streams)) if return_layers else logits
