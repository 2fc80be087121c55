"""Descriptions of parts: what a layer is made of, as data.

A model is a list of block descriptions and a schedule.  Each description names the
kind of part (looked up in `tau_rs_b200.parts.registry`) and carries every size and
constant that the part needs, so no part reads a model-wide configuration and none
knows which architecture it serves.  tau.rs expresses the same idea with one enum per
layer (crates/models/src/qwen3_5_common/decoder.rs:22-25,59-78: each layer owns either
kind of token mixer and its own state).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """`kind == "rms_norm"`: `x / sqrt(mean(x^2) + eps) * w`.  `kind == "layer_norm"`: `(x - mean) / sqrt(variance + eps) * w + b`,
    the bias being the tensor `<weight's name><bias_suffix>`.  With `groups` > 1 an RMS norm cuts the row into that many equal
    consecutive pieces and divides each by its own root mean square (on a residual stream kept in 32-bit)."""

    width: int
    eps: float
    kind: str = "rms_norm"
    bias_suffix: str = ".bias"
    bias: bool = True          # a layer norm without a bias has no such tensor
    groups: int = 1


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding of the first `rotary_dim` elements of each head."""

    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope_half"


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    bias: bool
    softmax_scale: float
    qk_norm: Optional[NormSpec] = None
    position: Optional[PositionSpec] = None
    window: Optional[int] = None
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    """`down(act(gate(x)) * up(x))` with `act` = `activation` ("silu" or "relu").  The three tensors are `<prefix>.<name><weight_suffix>`."""

    hidden: int
    intermediate: int
    kind: str = "swiglu"
    gate_name: str = "gate_proj"
    up_name: str = "up_proj"
    down_name: str = "down_proj"
    weight_suffix: str = ".weight"
    activation: str = "silu"


@dataclass(frozen=True)
class PairRotationSpec:
    """Rotary position encoding of the first `rotary_dim` elements of a vector in which element `2i` is paired with
    `2i + 1` (the interleaved layout); the angle of pair `i` at position `p` is `p * theta^(-2i / rotary_dim)`."""

    rotary_dim: int
    theta: float
    kind: str = "rope_pairs"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose keys and values are expanded from a cached latent of `kv_rank` elements per position, with
    `rot_dim` rotated key elements per position that all heads share, queries through a latent of `q_rank` elements, an
    optional learned sink per head in the softmax denominator and an optional sigmoid output gate."""

    hidden: int
    n_heads: int
    head_dim: int          # unrotated query/key elements per head
    rot_dim: int           # rotated query/key elements per head (the key's are shared by the heads)
    value_dim: int
    q_rank: int
    kv_rank: int
    softmax_scale: float
    eps: float             # of the two latent norms
    position: Optional[PairRotationSpec] = None
    sink: bool = True
    gate: bool = True
    window: Optional[int] = None
    kind: str = "latent_attention"


@dataclass(frozen=True)
class DifferentialAttentionSpec:
    """Softmax attention with two maps per head: each head has two queries and each key/value head two keys of `dim` elements
    (laid out head by head as [map 1, map 2]) over one value of `value_dim` elements; a head's result is
    `map 1 - lambda * map 2` with `lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff` (four learned vectors of `dim` elements, one
    number for the layer), divided by its root mean square over `value_dim` (eps inside the root, no weight), times `1 - diff`.
    Queries and keys pass an RMS norm over `dim` whose weight all heads and maps share, then `position`; `window` limits how far
    back a query sees (itself and the `window - 1` positions before it); `gate` multiplies the heads by a sigmoid of one more
    projection of the input before the output projection."""

    hidden: int
    n_heads: int
    n_kv_heads: int
    dim: int
    value_dim: int
    softmax_scale: float
    diff: float
    eps: float
    position: Optional[PairRotationSpec] = None
    window: Optional[int] = None
    gate: bool = True
    kind: str = "differential_attention"


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    """`down(act(up(x) + b_up)) + b_down` with `act` one of "relu_squared".  Tensors `<prefix>.<name><weight_suffix>` and, with
    `bias`, `<prefix>.<name><bias_suffix>`."""

    hidden: int
    intermediate: int
    activation: str = "relu_squared"
    bias: bool = True
    up_name: str = "up"
    down_name: str = "down"
    weight_suffix: str = ""
    bias_suffix: str = ".b"
    kind: str = "dense_mlp"


@dataclass(frozen=True)
class TokenSideSpec:
    """A per-layer input looked up by token id: `e` = columns `offset .. offset + dim` of the model's shared table `table`
    ([vocab, table_width]) at the token; `y = proj(gelu_tanh(gate(x)) * e)`; `x <- x + y / sqrt(mean(y^2) + eps) * w`."""

    table: str
    table_width: int
    offset: int
    dim: int
    eps: float


@dataclass(frozen=True)
class LinearRecurrenceSpec:
    """A matrix state per head, `S_t = a_t S_(t-1) + b_t k_t v_t^T`, read as `S_t^T q_t`.

    `gating == "decay"`: `a_t` is the head's constant of `decays`, `b_t = 1`, and q, k, v pass through `activation`.
    `gating == "exponential"`: a log input gate and a log forget gate per head and token (both soft-capped at `gate_cap`),
    a running maximum that keeps the exponentials in range, a normaliser state, and queries scaled by `query_scale`.
    `norm_groups` says over what the output is divided by its root mean square before the weight and the sigmoid gate:
    `"head"` (each head alone) or `"all"` (the concatenated heads)."""

    hidden: int
    n_heads: int
    key_dim: int
    value_dim: int
    gating: str
    eps: float
    norm_groups: str
    decays: Tuple[float, ...] = ()
    gate_cap: float = 0.0
    query_scale: float = 1.0
    activation: Optional[str] = None
    kind: str = "linear_recurrence"


@dataclass(frozen=True)
class ScaledRotationSpec:
    """Rotary position encoding of the first `rotary_dim` elements of each head in which element `i` is paired with element
    `i + rotary_dim / 2`; the angle of pair `i` at position `p` is `p * f_i` with `f_i = theta^(-2i / rotary_dim)`.  With `factor`
    (not None) the frequencies are blended between `f_i` and `f_i / factor` (YaRN): with `index(t) = rotary_dim * ln(original /
    (2 pi t)) / (2 ln theta)`, `lo = max(floor(index(fast)), 0)`, `hi = min(ceil(index(slow)), rotary_dim - 1)` and `ramp_i =
    clamp((i - lo) / max(hi - lo, 0.001), 0, 1)` the frequency is `f_i / factor * ramp_i + f_i * (1 - ramp_i)`, and sine and cosine
    are multiplied by `0.1 ln(factor) + 1`."""

    rotary_dim: int
    theta: float
    factor: Optional[float] = None
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0
    kind: str = "rope_half_scaled"


@dataclass(frozen=True)
class MaskedAttentionSpec:
    """Grouped-query softmax attention whose keys (`dim`) and values (`value_dim`) may differ in size, over one cached row per
    position (or over pages of ordinary heads where the sizes allow the tensor-core kernel).  `qk_norm == "projection"`: queries, and keys, pass an RMS norm over their whole projection (all heads at once) with a
    weight of that size, before `position`.  A query at position i sees key j <= i within `window` positions, or (with `chunk`)
    only if floor(j / chunk) == floor(i / chunk), chunks counted from position 0.  `sink`: one is added to the softmax's
    denominator (a key with score 0 and no value).  `out_scale` multiplies what the output projection reads.

    `bias`: q, k and v have biases (`<name>.b`).  `taps` > 0: q, k and v each pass a causal convolution of that many taps over time
    per channel directly behind the projection (`<name>.conv` [channels, taps], no bias, no activation), whose last `taps - 1`
    inputs are state of the sequence.  `temperature` = (coef, every): the query at position p is multiplied by
    `1 + coef * ln(floor((p + 1) / every) + 1)`.  `distance_bias`: `r1 * ln(1 + r2 * (i - j))` is taken off the score, with one r1 and
    one r2 per head (`r1`, `r2`).  `weights == "sigmoid"`: no softmax; a visible key weighs `sigmoid(score + pb[head])` (`pb`, one
    number per head), not normalised over the keys.  `gate`: `"head"` multiplies each head's result by the sigmoid of one number per
    head, `"element"` every element by the sigmoid of its own (`g`, a projection of the mixer's input).  `own_keys=False`: the
    layer has no key and value tensors and reads the keys and values that another layer of the same sizes cached."""

    hidden: int
    n_heads: int
    n_kv_heads: int
    dim: int
    value_dim: int
    softmax_scale: float
    eps: float = 1e-6
    qk_norm: Optional[str] = None
    position: Optional[ScaledRotationSpec] = None
    window: Optional[int] = None
    chunk: Optional[int] = None
    sink: bool = False
    kind: str = "masked_attention"
    bias: bool = False
    taps: int = 0
    temperature: Optional[Tuple[float, int]] = None
    distance_bias: bool = False
    weights: str = "softmax"
    gate: Optional[str] = None
    own_keys: bool = True


@dataclass(frozen=True)
class DeltaRuleSpec:
    """The gated delta rule: per head a matrix state `S` (`key_dim` x `value_dim`), `S <- g S; u = beta (v - S^T k); S <- S + k
    u^T; o = S^T q`.  Queries and keys belong to `n_key_heads` heads (value head h reads key head h / (n_heads / n_key_heads)).
    q, k and v each pass a causal convolution of `taps` taps per channel and SiLU; q and k are then unit vectors per head, q times
    `key_dim^-1/2`; `beta = sigmoid(W_b h)`; `g = exp(-exp(A_log) softplus(W_a h + dt_bias))`.  Each head's read-out is divided by
    its root mean square (`eps`), times a weight of `value_dim` elements shared by the heads, times `silu(W_g h)`.

    `decay == "channel"`: g is a vector over the state's rows, one decay per head and key channel, from pre-activations laid out
    heads x key_dim (`dt_bias` is then as wide; `A_log` stays one number per head).  `decay_rank` > 0: the decay's pre-activation is
    `W_a2 (W_a1 h)` through that many numbers (`a1`, `a2`) instead of `W_a h`; `gate_rank` > 0 likewise `W_g2 (W_g1 h)` (`g1`, `g2`)
    for the output gate.  `gate_activation`: `"silu"` or `"sigmoid"`."""

    hidden: int
    n_heads: int
    n_key_heads: int
    key_dim: int
    value_dim: int
    taps: int
    eps: float
    kind: str = "gated_delta_rule"
    decay: str = "head"
    decay_rank: int = 0
    gate_rank: int = 0
    gate_activation: str = "silu"


@dataclass(frozen=True)
class ChannelDecayMemorySpec:
    """Time mixing with a matrix state per head (`key_dim` x `key_dim`), a decay per key channel and a bonus for the token itself:
    with h' the input of the token before (zeros for the first token) every projection reads its own mix `h + (h' - h) * mu_s`;
    `r`, `k`, `v` are projections of their mixes, `gate = silu(W_g mix_g)`, `w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))` through
    `decay_rank` numbers; per head `o = (S + diag(u) k v^T)^T r`, then `S <- diag(w) S + k v^T`; each head's `o` is divided by its
    root mean square (`eps`), times `norm`, times the gate, then `W_o`."""

    hidden: int
    n_heads: int
    key_dim: int
    decay_rank: int
    eps: float
    kind: str = "channel_decay_memory"


@dataclass(frozen=True)
class SelectiveScanSpec:
    """A Mamba mixer: `[x | z] = W_in h`; x passes a causal convolution of `taps` taps per channel (with bias) and SiLU;
    `[dt | B | C] = W_x x` (`dt_rank`, `states`, `states`); `step = softplus(W_dt dt + b_dt)`; per channel and state
    `S <- exp(step A) S + step x B`, `y = S . C + D x` with `A = -exp(A_log)`; the output is `W_o (y silu(z))`."""

    hidden: int
    inner: int
    states: int
    dt_rank: int
    taps: int
    kind: str = "selective_scan"


@dataclass(frozen=True)
class SideBySideSpec:
    """Two mixers that read the same input; the result is `left_scale * left(h) + right_scale * right(h)`.  Their tensors lie under
    `<prefix>.<left_name>` and `<prefix>.<right_name>`.  `join == "normed"`: each side's result is first divided by its root mean
    square over the model width (`eps`) and multiplied by a weight of its own (`<prefix>.<side name>.out`)."""

    left: object
    right: object
    left_scale: float = 1.0
    right_scale: float = 1.0
    left_name: str = "left"
    right_name: str = "right"
    kind: str = "side_by_side"
    join: str = "sum"
    eps: float = 0.0


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """`top` of `experts` gated feed-forwards per token.  The router's logits pass through `score` ("sigmoid" or
    "softmax"); experts are chosen by score plus a correction per expert (if `correction`), weighted by the score itself,
    renormalised over the chosen ones only if `renormalize` (a softmax score renormalised is the softmax over the chosen logits
    alone).  `router_bias` adds the tensor `<prefix>.router.b` to the logits.  `weigh` says what an expert's weight multiplies:
    its `"output"`, or its `"input"` (the expert then reads `weight * h`).  `shared` is a feed-forward that every token passes; with
    `shared_gate` its output is scaled by the sigmoid of one more projection of the token.  `identity` > 0: the router has that
    many more outputs, behind the experts', which stand for experts without tensors that return what they read."""

    hidden: int
    intermediate: int
    experts: int
    top: int
    score: str = "sigmoid"
    correction: bool = True
    renormalize: bool = False
    shared: Optional[SwiGLUSpec] = None
    shared_gate: bool = False
    kind: str = "routed_experts"
    router_bias: bool = False
    weigh: str = "output"
    identity: int = 0


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its weight-name prefix, its two parts and the norm before each.  `residual_scale` (parallel blocks): what the two
    parts return is multiplied by it as it joins the residual stream."""

    prefix: str
    mixer: object
    feed_forward: object
    mixer_norm: NormSpec
    feed_forward_norm: Optional[NormSpec]
    kind: str = "pre_norm"
    residual_scale: float = 1.0


@dataclass(frozen=True)
class SublayerNormBlockSpec:
    """One layer whose norms act on what a sublayer returns: `x <- x + norm(gate * mixer(read(x)))`, then the same with the
    feed-forward (absent if `feed_forward` is None), on a residual stream kept in 32-bit; both sublayers read `x` itself.

    `input_taps` > 0: the mixer reads `x + conv(x)`, a causal convolution of that many taps over time on each channel, whose last
    `input_taps - 1` inputs are state of the sequence.  `residual_gate`: each sublayer's result is multiplied by
    `sigmoid(W x + b)` before its norm.  `token_side`: a per-layer input by token id joins the stream after the feed-forward.
    `depth_mix` = n > 0: what the block hands on is `sum_j w[j] * X_j` over the model's first n results (`X_0` the embedding
    output, `X_(k+1)` what run k of the schedule produced before this mixing), n being this run's index plus 2."""

    prefix: str
    mixer: object
    feed_forward: object
    mixer_norm: NormSpec
    feed_forward_norm: Optional[NormSpec]
    input_taps: int = 0
    residual_gate: bool = False
    token_side: Optional[TokenSideSpec] = None
    depth_mix: int = 0
    kind: str = "sublayer_norm"


@dataclass(frozen=True)
class SandwichBlockSpec:
    """One layer with a norm before and behind each sublayer, on a residual stream kept in 32-bit:
    `x <- x + s1 * post1(mixer(pre1(x)))`, then `x <- x + s2 * post2(feed_forward(pre2(x)))` (absent without a feed-forward).
    With `layer_scale` the vectors `s1`, `s2` (`<prefix>.<scale names>`) multiply the normalised results element by element."""

    prefix: str
    mixer: object
    feed_forward: object
    mixer_norm: NormSpec
    mixer_post_norm: NormSpec
    feed_forward_norm: Optional[NormSpec]
    feed_forward_post_norm: Optional[NormSpec]
    layer_scale: bool = True
    kind: str = "sandwich"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    `layer` indexes the model's blocks (a block may be named by several entries and
    then runs several times with the same weights).  `cache_group` and `cache_layer`
    say where the mixer keeps what it remembers; two entries with the same pair share
    that storage, and an entry with `writes_cache=False` only reads what another entry
    wrote earlier in the same step.
    """

    layer: int
    cache_group: Optional[str] = None
    cache_layer: int = 0
    writes_cache: bool = True
    # What the block keeps beside its mixer's cache (`Block.extra_cache_needs()`): (role, cache group, cache layer) for each role.
    extra_cache: Tuple[Tuple[str, str, int], ...] = ()


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    max_positions: int
    embedding_name: str
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    final_norm_name: str
    head_name: str
    tie_head: bool
    declared_dtype: Optional[str] = None
    extra: dict = field(default_factory=dict, compare=False)
    # A position encoding that acts on the embedded tokens before the first block (learned or absolute positions): a spec of
    # the "position" family whose part offers `add_to(hidden, step)`.  None for encodings that act inside the mixers.
    input_position: Optional[object] = None
    # "float32": the residual stream is kept in 32-bit whatever the run's dtype (None: in the run's dtype).
    residual_dtype: Optional[str] = None
    # The model keeps the embedding output and the result of every run of the schedule for the step's tokens
    # (`StepContext.results` [runs + 1, tokens, hidden]; `StepContext.run` is the index of the run that is being computed).
    keeps_results: bool = False
    # Tensors that belong to no single block: (name, shape, role).  The model reads them and hands each to the blocks that
    # list its name in `shared_tensor_names()`.
    shared_tensors: Tuple[Tuple[str, Tuple[int, ...], str], ...] = ()
    # The embedded rows are multiplied by this as they enter the residual stream (a 32-bit stream if it is not 1); the head reads
    # the table as it is.
    embedding_scale: float = 1.0
    # The logits are the head's product times this.
    logit_scale: float = 1.0
