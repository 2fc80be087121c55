"""Routed experts: each token passes `top` of `experts` gated feed-forwards, and optionally a shared one.

    z = W_router h (+ b_router) (32-bit);   s = sigmoid(z) (or softmax(z))
    chosen = the `top` experts with the largest s + correction;   weights = s of the chosen (renormalised only if asked)
    out = sum over chosen e of weight_e * W_down,e (silu(W_gate,e h) * (W_up,e h))  +  sigmoid(w_sg . h) * shared(h)
    (`weigh == "input"`: the weight multiplies what the expert reads instead, out = sum over chosen e of expert_e(weight_e * h))

The router, the choice and the weighted sum are 32-bit, and so is the output.  The experts' weights are stacked
(`[experts, 2 I, width]`, `[experts, width, I]`).  Two ways through the experts:

* few tokens (every decode step, and all of float32): weight-streaming kernels that index the experts by the router's choice
  on the device; nothing travels to the host, so a decode step through this part is captured in a graph like any other;
* runs of new tokens in bfloat16 (`GROUPED_FROM` pairs or more): the (token, place) pairs are grouped by expert on the
  device, each expert's rows pass through the tensor-core products that dense feed-forwards use (gate and up as one gated
  product), and a last kernel sums each token's places in place order.  The host reads the experts' row counts for this
  (one small copy per layer), which a prompt's step can afford and a captured decode step could not.

`identity` experts have no tensors: the router scores them like the others (its last outputs), and a token that chooses one adds
its weight times the token itself.  The expert kernels skip such places and the summing kernels put the token's row in their stead.

Both compute the same sums in 32-bit from the same roundings of the inputs; they differ as two product kernels differ.
A step reads only the experts that its tokens chose, which `bytes_read_per_step` accounts for.  Tensor names under the
prefix: `router`, `router.b`, `correction`, `e<j>.gate`, `e<j>.up`, `e<j>.down`, `shared.gate|up|down`, `shared.sg`.
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import FeedForward
from .registry import build, register_feed_forward


GROUPED_FROM = 512    # (token, place) pairs from which a run of new tokens takes the grouped products


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, spec, prefix: str, dtype, device):
        if spec.score not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown router score {spec.score!r}")
        if spec.top < 1 or spec.experts < 1:
            raise ValueError("top and the number of experts must be positive")
        if getattr(spec, "weigh", "output") not in ("output", "input"):
            raise ValueError(f"the experts' weights act on their output or their input, not on {spec.weigh!r}")
        if spec.shared_gate and spec.shared is None:
            raise ValueError("a shared gate needs a shared expert")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        self.identity = getattr(spec, "identity", 0)
        if self.identity < 0:
            raise ValueError("the number of identity experts cannot be negative")
        if self.identity and getattr(spec, "weigh", "output") == "input":
            raise ValueError("identity experts are summed with their weights on the output; weights on the experts' input are not served beside them")
        self.outputs = spec.experts + self.identity      # what the router scores
        if spec.top > self.outputs:
            raise ValueError("top must lie between 1 and the number of router outputs")
        self.shared = None if spec.shared is None else build("feed_forward", spec.shared, prefix=f"{prefix}.shared", dtype=dtype, device=device)
        self._own = {f"{prefix}.router": TensorSpec((self.outputs, spec.hidden), role="vector")}
        if spec.correction:
            self._own[f"{prefix}.correction"] = TensorSpec((self.outputs,), role="vector")
        if getattr(spec, "router_bias", False):
            self._own[f"{prefix}.router.b"] = TensorSpec((self.outputs,), role="vector")
        if spec.shared_gate:
            self._own[f"{prefix}.shared.sg"] = TensorSpec((1, spec.hidden), role="vector")
        for expert in range(spec.experts):
            self._own[f"{prefix}.e{expert}.gate"] = TensorSpec((spec.intermediate, spec.hidden), role="matrix")
            self._own[f"{prefix}.e{expert}.up"] = TensorSpec((spec.intermediate, spec.hidden), role="matrix")
            self._own[f"{prefix}.e{expert}.down"] = TensorSpec((spec.hidden, spec.intermediate), role="matrix")
        # Where the gated product exists the experts' gate and up rows are interleaved for it (as a dense feed-forward's are).
        self.interleave = kernels.GATE_GROUP if kernels.gated_fits(spec.hidden, spec.intermediate, dtype) and spec.intermediate % 8 == 0 else 0
        self._held = {}
        self.router = self.router_bias = self.correction = self.shared_gate = self.gate_up = self.down = None

    def tensor_specs(self):
        specs = dict(self._own)
        if self.shared is not None:
            specs.update(self.shared.tensor_specs())
        return specs

    def assign(self, name, tensor):
        if name in self._own:
            self._held[name] = tensor
        elif self.shared is not None:
            self.shared.assign(name, tensor)
        else:
            raise KeyError(name)

    def finalize_weights(self):
        spec, prefix, held = self.spec, self.prefix, self._held
        if self.shared is not None:
            self.shared.finalize_weights()
        self.router = held.pop(f"{prefix}.router")
        self.correction = held.pop(f"{prefix}.correction") if spec.correction else None
        self.router_bias = held.pop(f"{prefix}.router.b") if getattr(spec, "router_bias", False) else None
        self.shared_gate = held.pop(f"{prefix}.shared.sg").reshape(-1).contiguous() if spec.shared_gate else None
        group = self.interleave

        def stacked(gate, up):
            if not group:
                return torch.cat([gate, up], dim=0)
            return torch.stack([gate.view(-1, group, spec.hidden), up.view(-1, group, spec.hidden)], dim=1).reshape(-1, spec.hidden)

        self.gate_up = torch.stack([stacked(held.pop(f"{prefix}.e{e}.gate"), held.pop(f"{prefix}.e{e}.up")) for e in range(spec.experts)])
        self.down = torch.stack([held.pop(f"{prefix}.e{e}.down") for e in range(spec.experts)])

    def bytes_read_per_step(self, dtype) -> int:
        """The router, the shared expert and `top` experts: what a step of one token reads (more tokens read more experts,
        at most all of them)."""
        spec = self.spec
        element = torch.empty((), dtype=dtype).element_size()
        total = self.outputs * spec.hidden * 4 + min(spec.top, spec.experts) * 3 * spec.intermediate * spec.hidden * element
        return total + (self.shared.bytes_read_per_step(dtype) if self.shared is not None else 0)

    def forward(self, hidden, step):
        spec = self.spec
        tokens, device = hidden.shape[0], hidden.device
        chosen = torch.empty((tokens, spec.top), dtype=torch.int32, device=device)
        weights = torch.empty((tokens, spec.top), dtype=torch.float32, device=device)
        shared_gate = torch.empty((tokens,), dtype=torch.float32, device=device) if spec.shared_gate else None
        kernels.moe_route(hidden, self.router, self.correction, self.shared_gate, chosen, weights, shared_gate, spec.top,
                          spec.score == "softmax", spec.renormalize, self.router_bias)
        shared_out = None if self.shared is None else self.shared.forward(hidden, step)
        out = torch.empty((tokens, spec.hidden), dtype=torch.float32, device=device)
        if self.interleave and not step.all_single and tokens * spec.top >= GROUPED_FROM and not torch.cuda.is_current_stream_capturing():
            self._grouped(hidden, chosen, weights, shared_out, shared_gate, out)
            return out
        inner = torch.empty((tokens, spec.top, spec.intermediate), dtype=hidden.dtype, device=device)
        on_input = getattr(spec, "weigh", "output") == "input"
        kernels.moe_gate_up(hidden, self.gate_up, chosen, inner, self.interleave, weights if on_input else None)
        kernels.moe_down(inner, self.down, chosen, None if on_input else weights, shared_out, shared_gate, out, hidden if self.identity else None)
        return out

    def _grouped(self, hidden, chosen, weights, shared_out, shared_gate, out) -> None:
        spec = self.spec
        pairs, device = chosen.numel(), hidden.device
        offsets = torch.empty(self.outputs + 1, dtype=torch.int32, device=device)
        order = torch.empty(pairs, dtype=torch.int32, device=device)
        position = torch.empty(pairs, dtype=torch.int32, device=device)
        kernels.moe_sort(chosen, self.outputs, offsets, order, position)
        bounds = offsets.tolist()[: spec.experts + 1]    # the host waits here for the router; identity experts' pairs lie behind and have no product
        gathered = torch.empty((pairs, spec.hidden), dtype=hidden.dtype, device=device)
        on_input = getattr(spec, "weigh", "output") == "input"
        kernels.moe_gather(hidden, order, spec.top, gathered, weights if on_input else None)
        inner = torch.empty((pairs, spec.intermediate), dtype=hidden.dtype, device=device)
        rows = torch.empty((pairs, spec.hidden), dtype=torch.float32, device=device)
        kernels.gemm_tc_groups(gathered, self.gate_up, inner, bounds, gated=True)
        kernels.gemm_tc_groups(inner, self.down, rows, bounds)
        if self.identity:
            kernels.moe_combine(rows, position, None if on_input else weights, shared_out, shared_gate, out, chosen, hidden, spec.experts)
        else:
            kernels.moe_combine(rows, position, None if on_input else weights, shared_out, shared_gate, out)
