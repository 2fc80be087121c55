"""Pegurax stated plainly: one function per mechanism, float64, whole sequences, masks instead of caches, loops over tokens
instead of carried state.

Shares nothing with the library.  `weights` maps tensor names to float64 tensors, `config` is the dictionary that a folder's
config.json holds.  Every function takes one sequence `[tokens, ...]` whose first row is position 0.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def layer_norm(x, weight, eps):
    mean = x.mean(-1, keepdim=True)
    deviation = x - mean
    return deviation / torch.sqrt((deviation * deviation).mean(-1, keepdim=True) + eps) * weight


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_convolution(x, taps_weight, bias=None):
    """`out[t, c] = sum_j w[c, j] * x[t - (taps - 1) + j, c]`: the last column weighs the token itself, rows before the start are zero."""
    tokens = x.shape[0]
    taps = taps_weight.shape[1]
    out = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < tokens:
            out[back:] += taps_weight[:, j] * x[: tokens - back]
    return out if bias is None else out + bias


def scaled_frequencies(rot):
    """Per pair: the frequency after the blend between the original and the slowed-down one, and the factor on sine and cosine."""
    dims, base = rot["dims"], rot["base"]
    plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if scaling is None:
        return plain, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def turns_to_index(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    low = max(math.floor(turns_to_index(scaling["fast"])), 0)
    high = min(math.ceil(turns_to_index(scaling["slow"])), dims - 1)
    out = []
    for i, f in enumerate(plain):
        ramp = min(max((i - low) / max(high - low, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_halves(x, rot, first_position=0):
    """`x` [tokens, heads, dim]: element i of the first `dims` is paired with element i + dims / 2."""
    dims = rot["dims"]
    if dims == 0:
        return x
    half = dims // 2
    frequencies, magnitude = scaled_frequencies(rot)
    positions = torch.arange(first_position, first_position + x.shape[0], dtype=F).view(-1, 1, 1)
    angle = positions * torch.tensor(frequencies, dtype=F).view(1, 1, half)
    cos, sin = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def chunked_sink_attention(q, k, v, scale, chunk):
    """One head: token i sees j <= i of its own chunk of `chunk` positions; the softmax's denominator has one added."""
    tokens = q.shape[0]
    i, j = torch.arange(tokens).view(-1, 1), torch.arange(tokens).view(1, -1)
    scores = (q @ k.T) * scale
    hidden = (j > i) | (i // chunk != j // chunk)
    scores = scores.masked_fill(hidden, float("-inf"))
    top = torch.clamp(scores.max(-1, keepdim=True).values, min=0.0)
    weights = torch.exp(scores - top)
    return (weights / (torch.exp(-top) + weights.sum(-1, keepdim=True))) @ v


def softmax_branch(h, weights, prefix, mixer, eps):
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    tokens = h.shape[0]
    q = unit_rms(h @ weights[f"{prefix}.q"].T, eps) * weights[f"{prefix}.q.norm"]          # over the whole projection
    k = unit_rms(h @ weights[f"{prefix}.k"].T, eps) * weights[f"{prefix}.k.norm"]
    v = (h @ weights[f"{prefix}.v"].T).view(tokens, kv_heads, vdim)
    q = rotate_halves(q.view(tokens, heads, dim), mixer["rot"])
    k = rotate_halves(k.view(tokens, kv_heads, dim), mixer["rot"])
    out = torch.zeros((tokens, heads, vdim), dtype=F)
    for head in range(heads):
        group = head // (heads // kv_heads)
        out[:, head] = chunked_sink_attention(q[:, head], k[:, group], v[:, group], mixer["scale"], mixer["mask"]["size"])
    return out.reshape(tokens, heads * vdim) @ weights[f"{prefix}.o"].T


def gated_delta_rule(q, k, v, beta, decay):
    """One head: `q`, `k` [tokens, dim], `v` [tokens, vdim], `beta`, `decay` [tokens]; the state starts at zero."""
    tokens, dim = q.shape
    state = torch.zeros((dim, v.shape[1]), dtype=F)
    out = torch.zeros_like(v)
    for t in range(tokens):
        state = decay[t] * state
        update = beta[t] * (v[t] - state.T @ k[t])
        state = state + torch.outer(k[t], update)
        out[t] = state.T @ q[t]
    return out


def delta_branch(h, weights, prefix, mixer, eps):
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    tokens = h.shape[0]

    def through(name):
        return silu(causal_convolution(h @ weights[f"{prefix}.{name}"].T, weights[f"{prefix}.{name}.conv"]))

    def unit(x):
        return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)

    q = unit(through("q").view(tokens, kv_heads, dim)) * dim ** -0.5
    k = unit(through("k").view(tokens, kv_heads, dim))
    v = through("v").view(tokens, heads, vdim)
    beta = torch.sigmoid(h @ weights[f"{prefix}.b"].T)
    decay = torch.exp(-torch.exp(weights[f"{prefix}.A_log"]) * softplus(h @ weights[f"{prefix}.a"].T + weights[f"{prefix}.dt_bias"]))
    out = torch.zeros((tokens, heads, vdim), dtype=F)
    for head in range(heads):
        group = head // (heads // kv_heads)
        out[:, head] = gated_delta_rule(q[:, group], k[:, group], v[:, head], beta[:, head], decay[:, head])
    out = unit_rms(out, eps) * weights[f"{prefix}.norm"]
    out = out.reshape(tokens, heads * vdim) * silu(h @ weights[f"{prefix}.g"].T)
    return out @ weights[f"{prefix}.o"].T


def parallel_mixer(h, weights, prefix, mixer, eps):
    return (mixer["left_scale"] * softmax_branch(h, weights, f"{prefix}.left", mixer["left"], eps)
            + mixer["right_scale"] * delta_branch(h, weights, f"{prefix}.right", mixer["right"], eps))


def selective_scan_mixer(h, weights, prefix, mixer):
    inner, states, rank = mixer["inner"], mixer["state"], mixer["dt_rank"]
    tokens = h.shape[0]
    both = h @ weights[f"{prefix}.in"].T
    x, z = both[:, :inner], both[:, inner:]
    x = silu(causal_convolution(x, weights[f"{prefix}.conv"], weights[f"{prefix}.conv.b"]))
    low = x @ weights[f"{prefix}.x"].T
    step = softplus(low[:, :rank] @ weights[f"{prefix}.dt"].T + weights[f"{prefix}.dt.b"])          # [tokens, inner]
    b, c = low[:, rank : rank + states], low[:, rank + states :]
    a = -torch.exp(weights[f"{prefix}.A_log"])                                                     # [inner, states]
    state = torch.zeros((inner, states), dtype=F)
    y = torch.zeros((tokens, inner), dtype=F)
    for t in range(tokens):
        state = torch.exp(step[t].view(-1, 1) * a) * state + (step[t] * x[t]).view(-1, 1) * b[t].view(1, -1)
        y[t] = state @ c[t] + weights[f"{prefix}.D"] * x[t]
    return (y * silu(z)) @ weights[f"{prefix}.o"].T


def gated_feed_forward(h, weights, prefix, activation):
    return (activation(h @ weights[f"{prefix}.gate"].T) * (h @ weights[f"{prefix}.up"].T)) @ weights[f"{prefix}.down"].T


def routed_feed_forward(h, weights, prefix, mlp):
    """Sigmoid scores; the `top` largest are chosen and weigh the chosen experts' inputs as they are."""
    scores = torch.sigmoid(h @ weights[f"{prefix}.router"].T)
    chosen = torch.topk(scores, mlp["router"]["top"], dim=-1).indices
    out = torch.zeros_like(h)
    for token in range(h.shape[0]):
        for expert in chosen[token].tolist():
            row = (scores[token, expert] * h[token]).view(1, -1)
            out[token] += gated_feed_forward(row, weights, f"{prefix}.e{expert}", silu)[0]
    return out


def forward(tokens, weights, config, return_layers=False):
    """Logits `[tokens, vocab]` of one sequence; with `return_layers` also the residual stream after every layer."""
    eps = config["norm"]["eps"]
    x = weights["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    kept = []
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}"
        h = layer_norm(x, weights[f"{prefix}.norm1"], eps)
        if layer["type"] == "parallel":
            mixed = parallel_mixer(h, weights, f"{prefix}.mix", layer["mixer"], eps)
        else:
            mixed = selective_scan_mixer(h, weights, f"{prefix}.mix", layer["mixer"])
        x = x + layer_norm(mixed, weights[f"{prefix}.norm1b"], eps) * weights[f"{prefix}.ls1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, weights[f"{prefix}.norm2"], eps)
            if mlp["kind"] == "dense":
                fed = gated_feed_forward(h, weights, f"{prefix}.mlp", torch.relu)
            else:
                fed = routed_feed_forward(h, weights, f"{prefix}.mlp", mlp)
            x = x + layer_norm(fed, weights[f"{prefix}.norm2b"], eps) * weights[f"{prefix}.ls2"]
        kept.append(x)
    logits = layer_norm(x, weights["final.norm"], eps) @ weights["embed"].T
    return (logits, torch.stack(kept)) if return_layers else logits
