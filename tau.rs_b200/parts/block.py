"""Pre-norm block: `r = x + mixer(norm(x))`, `out = r + feed_forward(norm(r))`.

crates/models/src/qwen3_5_common/decoder.rs:96-117.  The hidden state travels as
`(residual, branch)` with `x = residual + branch`, so each sum is rounded to the storage
dtype and normalised by one fused kernel (crates/models/src/components/rms_norm.rs:39-74).
Weight names: `<prefix>.input_layernorm`, `<prefix>.self_attn`,
`<prefix>.post_attention_layernorm`, `<prefix>.mlp` (decoder.rs:52,296,302).
"""
from __future__ import annotations

import math

import torch

from ..csrc import kernels
from .base import Block
from .registry import build, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    mixer_name = "self_attn"
    feed_forward_name = "mlp"
    mixer_norm_name = "input_layernorm"
    feed_forward_norm_name = "post_attention_layernorm"

    def __init__(self, spec, dtype, device):
        self.spec = spec
        prefix = spec.prefix
        self.mixer_norm = build("norm", spec.mixer_norm, name=f"{prefix}.{self.mixer_norm_name}.weight", dtype=dtype, device=device)
        self.mixer = build("mixer", spec.mixer, prefix=f"{prefix}.{self.mixer_name}", dtype=dtype, device=device)
        self.feed_forward_norm = build(
            "norm", spec.feed_forward_norm, name=f"{prefix}.{self.feed_forward_norm_name}.weight", dtype=dtype, device=device
        )
        self.feed_forward = build(
            "feed_forward", spec.feed_forward, prefix=f"{prefix}.{self.feed_forward_name}", dtype=dtype, device=device
        )
        self._children = (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
        self.capturable = all(getattr(part, "capturable", True) for part in self._children)

    def cache_need(self):
        return self.mixer.cache_need()

    def decode_blocks(self):
        return self.mixer.decode_blocks()

    def tensor_specs(self):
        specs = {}
        for part in self._children:
            specs.update(part.tensor_specs())
        return specs

    def assign(self, name, tensor):
        for part in self._children:
            if name in part.tensor_specs():
                return part.assign(name, tensor)
        raise KeyError(name)

    def finalize_weights(self):
        for part in self._children:
            part.finalize_weights()

    def bytes_read_per_step(self, dtype) -> int:
        return sum(part.bytes_read_per_step(dtype) for part in self._children)

    def forward(self, residual, branch, step, cache, writes_cache: bool):
        if branch is None:
            normalized = self.mixer_norm.forward(residual)
        else:
            normalized = self.mixer_norm.add_forward(branch, residual)
        mixed = self.mixer.forward(normalized, step, cache, writes_cache)
        normalized = self.feed_forward_norm.add_forward(mixed, residual)
        return residual, self.feed_forward.forward(normalized, step)


@register_block("parallel")
class ParallelBlock(Block):
    """One norm, two readers: `h = norm(x)`, `x <- x + (mixer(h) + feed_forward(h))`; the feed-forward may be absent.

    The residual stream `x` is 32-bit whatever the activations' dtype.  The block hands on `(x, (mixer's output,
    feed-forward's output))`; the next block's norm (or the model's last one) adds the two in 32-bit, adds that to the
    stream and normalises, in one kernel.  With `residual_scale` m the sum joins as `x + m * (mixer(h) + feed_forward(h))`.
    What the mixer keeps beside its cache (`extra_cache_needs`) is the block's as well.  Weight names: `<prefix>.norm1`,
    `<prefix>.mix.*`, `<prefix>.mlp.*`.
    """

    mixer_name = "mix"
    feed_forward_name = "mlp"
    norm_name = "norm1"

    def __init__(self, spec, dtype, device):
        self.spec = spec
        prefix = spec.prefix
        self.norm = build("norm", spec.mixer_norm, name=f"{prefix}.{self.norm_name}", dtype=dtype, device=device)
        self.mixer = build("mixer", spec.mixer, prefix=f"{prefix}.{self.mixer_name}", dtype=dtype, device=device)
        self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward = build("feed_forward", spec.feed_forward, prefix=f"{prefix}.{self.feed_forward_name}", dtype=dtype, device=device)
        self._children = tuple(part for part in (self.norm, self.mixer, self.feed_forward) if part is not None)
        self.capturable = all(getattr(part, "capturable", True) for part in self._children)

    cache_need = PreNormBlock.cache_need
    decode_blocks = PreNormBlock.decode_blocks
    tensor_specs = PreNormBlock.tensor_specs
    assign = PreNormBlock.assign
    finalize_weights = PreNormBlock.finalize_weights
    bytes_read_per_step = PreNormBlock.bytes_read_per_step

    def extra_cache_needs(self):
        return self.mixer.extra_cache_needs()

    def forward(self, residual, branch, step, cache, writes_cache: bool):
        from .base import Pending

        normalized = self.norm.forward(residual) if branch is None else self.norm.add_forward(branch, residual)
        mixed = self.mixer.forward(normalized, step, cache, writes_cache)
        scale = getattr(self.spec, "residual_scale", 1.0)
        if self.feed_forward is None:
            return residual, (mixed if scale == 1.0 else Pending((mixed,), scale))
        return residual, Pending((mixed, self.feed_forward.forward(normalized, step)), scale)


@register_block("sublayer_norm")
class SublayerNormBlock(Block):
    """Norms on what the sublayers return, on a 32-bit residual stream `x`:

        read = x + conv(x)                          (a causal convolution over time per channel, if `input_taps`; else read = x)
        x <- x + norm1(sigmoid(W_g1 x + b_g1) * mixer(read))
        x <- x + norm2(sigmoid(W_g2 x + b_g2) * feed_forward(x))        (if there is a feed-forward)
        y = W_proj (gelu_tanh(W_gate x) * e[token]);  x <- x + y / rms(y) * w_side      (if `token_side`)
        X_(run + 1) = x;  handed on: sum_j mix[j] * X_j over the first `depth_mix` results     (if `depth_mix`)

    Each `x <- x + norm(...)` is one kernel that also rounds the new `x` for the products that read it next.  The convolution's
    last `input_taps - 1` inputs are state of the sequence (`extra_cache_needs()["taps"]`, 32-bit).  Weight names under the
    prefix: `norm1`, `norm2` (and their biases), `mix.*`, `mlp.*`, `canon1` [width, taps], `rg1`, `rg2` (with `.b`), `dwa`
    [depth_mix], `side.gate`, `side.proj`, `side.norm`.
    """

    mixer_name = "mix"
    feed_forward_name = "mlp"
    mixer_norm_name = "norm1"
    feed_forward_norm_name = "norm2"
    taps_name = "canon1"
    mixer_gate_name = "rg1"
    feed_forward_gate_name = "rg2"
    mix_name = "dwa"
    side_name = "side"

    def __init__(self, spec, dtype, device):
        from ..weights.tensor_spec import TensorSpec
        from .linear import StackedLinear

        self.spec, self.dtype = spec, dtype
        prefix, width = spec.prefix, spec.mixer_norm.width
        self.width = width
        self.mixer_norm = build("norm", spec.mixer_norm, name=f"{prefix}.{self.mixer_norm_name}", dtype=dtype, device=device)
        self.mixer = build("mixer", spec.mixer, prefix=f"{prefix}.{self.mixer_name}", dtype=dtype, device=device)
        self.feed_forward = self.feed_forward_norm = self.mixer_gate = self.feed_forward_gate = self.side_gate = self.side_proj = None
        if spec.feed_forward is not None:
            self.feed_forward = build("feed_forward", spec.feed_forward, prefix=f"{prefix}.{self.feed_forward_name}", dtype=dtype, device=device)
            self.feed_forward_norm = build("norm", spec.feed_forward_norm, name=f"{prefix}.{self.feed_forward_norm_name}", dtype=dtype, device=device)
        for norm in (spec.mixer_norm, spec.feed_forward_norm if spec.feed_forward is not None else None):
            if norm is not None and norm.kind not in ("layer_norm", "rms_norm"):
                raise ValueError(f"the block's kernel computes layer_norm and rms_norm; a norm of kind {norm.kind!r} is not served")
        names = dict(weight_suffix="", bias_suffix=".b")
        if spec.residual_gate:
            self.mixer_gate = StackedLinear([(f"{prefix}.{self.mixer_gate_name}", width)], width, True, dtype, device, **names)
            if self.feed_forward is not None:
                self.feed_forward_gate = StackedLinear([(f"{prefix}.{self.feed_forward_gate_name}", width)], width, True, dtype, device, **names)
        self._own = {}
        if spec.input_taps:
            self._own[f"{prefix}.{self.taps_name}"] = TensorSpec((width, spec.input_taps), role="vector", std=0.1)
        if spec.depth_mix:
            self._own[f"{prefix}.{self.mix_name}"] = TensorSpec((spec.depth_mix,), role="vector", std=0.5)
        side = spec.token_side
        if side is not None:
            self.side_gate = StackedLinear([(f"{prefix}.{self.side_name}.gate", side.dim)], width, False, dtype, device, **names)
            self.side_proj = StackedLinear([(f"{prefix}.{self.side_name}.proj", width)], side.dim, False, dtype, device, **names)
            self._own[f"{prefix}.{self.side_name}.norm"] = TensorSpec((width,), role="vector", init="ones")
        self._held = {}
        self.taps = self.mix = self.side_norm = self.side_table = None
        self._children = tuple(part for part in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward, self.mixer_gate,
                                                 self.feed_forward_gate, self.side_gate, self.side_proj) if part is not None)
        self.capturable = all(getattr(part, "capturable", True) for part in self._children)

    cache_need = PreNormBlock.cache_need
    decode_blocks = PreNormBlock.decode_blocks

    def extra_cache_needs(self):
        from .base import CacheNeed

        if self.spec.input_taps > 1:
            return {"taps": CacheNeed("state", state_shape=(self.spec.input_taps - 1, self.width))}
        return {}

    def shared_tensor_names(self):
        return () if self.spec.token_side is None else (self.spec.token_side.table,)

    def bind_shared(self, name, tensor):
        if self.spec.token_side is None or name != self.spec.token_side.table:
            raise KeyError(name)
        self.side_table = tensor

    def tensor_specs(self):
        specs = dict(self._own)
        for part in self._children:
            specs.update(part.tensor_specs())
        return specs

    def assign(self, name, tensor):
        if name in self._own:
            self._held[name] = tensor
            return
        for part in self._children:
            if name in part.tensor_specs():
                return part.assign(name, tensor)
        raise KeyError(name)

    def finalize_weights(self):
        prefix, spec = self.spec.prefix, self.spec
        for part in self._children:
            part.finalize_weights()
        # Stored [width, taps]; the kernel reads tap by tap, a tap's channels side by side.
        self.taps = self._held.pop(f"{prefix}.{self.taps_name}").t().contiguous() if spec.input_taps else None
        self.mix = self._held.pop(f"{prefix}.{self.mix_name}") if spec.depth_mix else None
        self.side_norm = self._held.pop(f"{prefix}.{self.side_name}.norm") if spec.token_side is not None else None

    def bytes_read_per_step(self, dtype) -> int:
        own = sum(4 * math.prod(spec.shape) for spec in self._own.values())
        return own + sum(part.bytes_read_per_step(dtype) for part in self._children)

    def _join(self, source, target, result, gate, norm, spec_norm, copy):
        kernels.gated_add_norm(source, target, result, gate, norm.weight, getattr(norm, "bias", None), spec_norm.eps, spec_norm.kind == "layer_norm", copy)

    def forward(self, residual, branch, step, cache, writes_cache: bool):
        spec = self.spec
        if branch is not None:
            raise ValueError("this block reads a finished stream; the block before it must not leave a branch pending")
        if residual.dtype != torch.float32:
            raise ValueError("this block keeps its residual stream in 32-bit (ModelSpec.residual_dtype)")
        x, shape, device = residual, residual.shape, residual.device
        # What the products read: the stream rounded once (`plain`), and for the mixer the stream plus its convolution (`read`).
        read = torch.empty(shape, dtype=self.dtype, device=device)
        plain = torch.empty(shape, dtype=self.dtype, device=device) if (spec.input_taps and spec.residual_gate) else None
        state = cache.extra["taps"].state if spec.input_taps > 1 else None
        kernels.causal_taps(x, self.taps, state, step, read, plain, update=writes_cache)
        mixed = self.mixer.forward(read, step, cache, writes_cache)
        gate = None if self.mixer_gate is None else self.mixer_gate.forward(read if plain is None else plain)
        if spec.depth_mix:
            if step.results is None or spec.depth_mix != step.run + 2:
                raise ValueError("the block mixes the model's results: the model must keep them, and this run must be number depth_mix - 2")
            target = step.results[step.run + 1]
        else:
            target = x
        rounded = torch.empty(shape, dtype=self.dtype, device=device)
        self._join(x, target, mixed, gate, self.mixer_norm, spec.mixer_norm, rounded)
        x = target
        if self.feed_forward is not None:
            fed = self.feed_forward.forward(rounded, step)
            gate = None if self.feed_forward_gate is None else self.feed_forward_gate.forward(rounded)
            after = torch.empty(shape, dtype=self.dtype, device=device)
            self._join(x, x, fed, gate, self.feed_forward_norm, spec.feed_forward_norm, after)
            rounded = after
        y = None
        if spec.token_side is not None:
            side = spec.token_side
            pre = self.side_gate.forward(rounded)
            kernels.side_gate(pre, self.side_table, step.token_ids, side.offset, pre)
            y = self.side_proj.forward(pre, out_dtype=torch.float32)
        if not spec.depth_mix:
            if y is not None:
                kernels.unit_add_mix(x, y, self.side_norm, spec.token_side.eps, x)
            return x, None
        out = torch.empty(shape, dtype=torch.float32, device=device)
        kernels.unit_add_mix(x, y, self.side_norm, 0.0 if y is None else spec.token_side.eps, x, step.results, self.mix, out)
        return out, None


@register_block("sandwich")
class SandwichBlock(Block):
    """A norm before and a norm behind each sublayer, on a 32-bit residual stream `x`:

        x <- x + s1 * post1(mixer(pre1(x)))
        x <- x + s2 * post2(feed_forward(pre2(x)))          (if there is a feed-forward)

    `s1`, `s2` are vectors of the stream's width (`layer_scale`); because the norms behind the sublayers have a weight and no bias,
    each is multiplied into its norm's weight once, when the weights are loaded.  A sublayer's result is normalised, added to the
    stream and the new stream normalised for the next reader by one kernel where the next reader is this block's own feed-forward.
    Weight names under the prefix: `norm1`, `norm1b`, `norm2`, `norm2b`, `ls1`, `ls2`, `mix.*`, `mlp.*`.
    """

    mixer_name = "mix"
    feed_forward_name = "mlp"
    norm_names = ("norm1", "norm1b", "norm2", "norm2b")
    scale_names = ("ls1", "ls2")

    def __init__(self, spec, dtype, device):
        from ..weights.tensor_spec import TensorSpec

        self.spec, self.dtype = spec, dtype
        prefix = spec.prefix
        self.width = spec.mixer_norm.width
        pre1, post1, pre2, post2 = (f"{prefix}.{name}" for name in self.norm_names)
        self.mixer_norm = build("norm", spec.mixer_norm, name=pre1, dtype=dtype, device=device)
        self.mixer_post_norm = build("norm", spec.mixer_post_norm, name=post1, dtype=dtype, device=device)
        self.mixer = build("mixer", spec.mixer, prefix=f"{prefix}.{self.mixer_name}", dtype=dtype, device=device)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = build("feed_forward", spec.feed_forward, prefix=f"{prefix}.{self.feed_forward_name}", dtype=dtype, device=device)
            self.feed_forward_norm = build("norm", spec.feed_forward_norm, name=pre2, dtype=dtype, device=device)
            self.feed_forward_post_norm = build("norm", spec.feed_forward_post_norm, name=post2, dtype=dtype, device=device)
        for norm in (spec.mixer_norm, spec.mixer_post_norm, spec.feed_forward_norm, spec.feed_forward_post_norm):
            if norm is None:
                continue
            if norm.kind not in ("layer_norm", "rms_norm"):
                raise ValueError(f"the block's kernels compute layer_norm and rms_norm; a norm of kind {norm.kind!r} is not served")
            if getattr(norm, "bias", True) and norm.kind == "layer_norm":
                raise ValueError("the block's norms have a weight and no bias")
        self._own = {}
        if spec.layer_scale:
            self._own[f"{prefix}.{self.scale_names[0]}"] = TensorSpec((self.width,), role="vector", init="ones")
            if self.feed_forward is not None:
                self._own[f"{prefix}.{self.scale_names[1]}"] = TensorSpec((self.width,), role="vector", init="ones")
        self._held = {}
        self.mixer_post_weight = self.feed_forward_post_weight = None
        self._children = tuple(part for part in (self.mixer_norm, self.mixer_post_norm, self.mixer, self.feed_forward_norm, self.feed_forward_post_norm,
                                                 self.feed_forward) if part is not None)
        self.capturable = all(getattr(part, "capturable", True) for part in self._children)

    cache_need = PreNormBlock.cache_need
    decode_blocks = PreNormBlock.decode_blocks
    tensor_specs = SublayerNormBlock.tensor_specs
    assign = SublayerNormBlock.assign

    def extra_cache_needs(self):
        return self.mixer.extra_cache_needs()

    def finalize_weights(self):
        prefix, spec = self.spec.prefix, self.spec
        for part in self._children:
            part.finalize_weights()
        self.mixer_post_weight = self.mixer_post_norm.weight
        self.feed_forward_post_weight = None if self.feed_forward is None else self.feed_forward_post_norm.weight
        if spec.layer_scale:
            self.mixer_post_weight = (self.mixer_post_weight * self._held.pop(f"{prefix}.{self.scale_names[0]}")).contiguous()
            if self.feed_forward is not None:
                self.feed_forward_post_weight = (self.feed_forward_post_weight * self._held.pop(f"{prefix}.{self.scale_names[1]}")).contiguous()

    def bytes_read_per_step(self, dtype) -> int:
        own = sum(4 * math.prod(spec.shape) for spec in self._own.values())
        return own + sum(part.bytes_read_per_step(dtype) for part in self._children)

    def forward(self, residual, branch, step, cache, writes_cache: bool):
        spec = self.spec
        if branch is not None:
            raise ValueError("this block reads a finished stream; the block before it must not leave a branch pending")
        if residual.dtype != torch.float32:
            raise ValueError("this block keeps its residual stream in 32-bit (ModelSpec.residual_dtype)")
        x = residual
        mixed = self.mixer.forward(self.mixer_norm.forward(x), step, cache, writes_cache)
        centred = spec.mixer_post_norm.kind == "layer_norm"
        if self.feed_forward is None:
            kernels.gated_add_norm(x, x, mixed, None, self.mixer_post_weight, None, spec.mixer_post_norm.eps, centred)
            return x, None
        kernels.gated_add_norm(x, x, mixed, None, self.mixer_post_weight, None, spec.mixer_post_norm.eps, centred)
        fed = self.feed_forward.forward(self.feed_forward_norm.forward(x), step)
        kernels.gated_add_norm(x, x, fed, None, self.feed_forward_post_weight, None, spec.feed_forward_post_norm.eps,
                               spec.feed_forward_post_norm.kind == "layer_norm")
        return x, None
