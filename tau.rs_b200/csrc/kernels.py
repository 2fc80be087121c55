"""Python face of the CUDA kernels: checks shapes and dtypes, then launches on the current stream.

Every function here runs a hand-written kernel of this folder; there is no other
implementation behind them.  If the extension cannot be compiled or loaded, or a tensor is
not on a CUDA device, the call fails with an error.  Kernels refuse sizes that they do not
cover instead of computing something else.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

PAGE_TOKENS = 64
_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _pointer(tensor: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream_handle() -> int:
    """The current stream of the current device as a number.  Asked of torch's C layer where it offers that: the Python-level
    `torch.cuda.current_stream()` costs several microseconds, and every launch asks."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _stream():
    return ctypes.c_void_p(_stream_handle())


def _code(tensor: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[tensor.dtype]
    except KeyError:
        raise KernelError(f"dtype {tensor.dtype} is not supported; use float32 or bfloat16") from None


def _require(condition: bool, message: str) -> None:
    if not condition:
        raise KernelError(message)


def _on_device(*tensors) -> None:
    for tensor in tensors:
        if tensor is not None:
            _require(tensor.is_cuda, "kernels run on CUDA tensors only; there is no CPU path")
            _require(tensor.is_contiguous() or tensor.stride(-1) == 1, "tensors must have a unit innermost stride")


_launches = 0
_replayed = 0


def launch_count() -> int:
    """Kernels of this library launched so far (those inside replayed graphs included)."""
    return _launches + _replayed


def count_replay(kernels_in_graph: int) -> None:
    global _replayed
    _replayed += kernels_in_graph


# Kernel classes for the timing of a step (crates/metrics/src/timing.rs:83-183 times the phases of a decode step with
# CUDA events): what each launch is booked under.
_CLASS_OF = {
    "embedding": "embedding", "rms_norm": "norm", "add_rms_norm": "norm", "silu_mul": "activation", "gemm_simt": "product",
    "gemm_skinny": "product", "gemm_tc": "product", "attention_prepare": "attention", "attention": "attention",
    "attention_decode": "attention", "attention_prefill": "attention", "attention_prefill_tc": "attention", "argmax": "selection",
    "sample_gumbel": "selection", "store_words_host": "selection", "random_normal": "other",
    "stream_add_norm": "norm", "normed_pair_sum": "norm", "gated_group_norm": "norm", "gemm_simt_batched": "product", "linear_recurrence": "recurrence",
    "latent_prepare": "attention", "latent_attention": "attention", "latent_expand": "attention", "moe_route": "routing", "moe_gate_up": "experts", "moe_down": "experts", "gemm_tc_groups": "experts", "moe_sort": "routing", "moe_gather": "routing",
    "moe_combine": "routing", "diff_prepare": "attention", "diff_attention": "attention", "diff_combine": "attention", "causal_taps": "norm", "gated_add_norm": "norm",
    "side_gate": "activation", "unit_add_mix": "norm", "norm_rows": "norm", "relu_squared": "activation",
    "short_conv": "recurrence", "delta_prepare": "recurrence", "delta_rule": "recurrence", "selective_scan": "recurrence",
    "masked_prepare": "attention", "masked_attention": "attention", "gated_rows": "attention",
    "token_shift": "recurrence", "tanh": "activation", "channel_decay": "recurrence", "wkv": "recurrence",
}
_timing = None     # while timing: [last event, [(class, event after the launch), ...]]


_timing_by_name = False


def start_timing(by_name: bool = False) -> None:
    """From now on an event follows every launch of this library on the current stream; `take_timing` reads them.
    Meant for steps that run outside a captured graph.  `by_name`: book every launch under its own name instead of its class."""
    global _timing, _timing_by_name
    _timing_by_name = by_name
    first = torch.cuda.Event(enable_timing=True)
    first.record()
    _timing = [first, []]


def take_timing(stop: bool = False) -> dict:
    """Milliseconds per kernel class since `start_timing` or the last `take_timing` (waits for the stream).  The time of
    a launch runs from the end of the launch before it, so gaps between kernels are booked to the kernel that follows."""
    global _timing
    if _timing is None:
        return {}
    first, marks = _timing
    totals = {}
    if marks:
        marks[-1][1].synchronize()
        previous = first
        for name, event in marks:
            totals[name] = totals.get(name, 0.0) + previous.elapsed_time(event)
            previous = event
        first = marks[-1][1]
    _timing = None if stop else [first, []]
    return {name: round(value, 4) for name, value in totals.items()}


def _check(status: int, what: str, kernels_launched: int = 1) -> None:
    global _launches
    _launches += kernels_launched
    if _timing is not None and status == 0 and not torch.cuda.is_current_stream_capturing():
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        _timing[1].append((what if _timing_by_name else _CLASS_OF.get(what, "other"), event))
    if status != 0:
        library = build.load_library("elementwise.cu")
        library.tau_error_string.restype = ctypes.c_char_p
        text = library.tau_error_string(ctypes.c_int(status)).decode()
        raise KernelError(f"{what} failed: {text} (CUDA error {status})")


def _f32_vector(tensor: Optional[torch.Tensor], length: int, what: str) -> None:
    if tensor is not None:
        _require(tensor.dtype == torch.float32 and tensor.numel() == length and tensor.is_contiguous(),
                 f"{what} must be a contiguous float32 vector of {length} elements")


def _int_vector(tensor: torch.Tensor, what: str) -> None:
    _require(tensor.dtype == torch.int32 and tensor.stride(-1) == 1, f"{what} must be int32")


# ---------------------------------------------------------------------------- elementwise
def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """`out[i] = table[tokens[i]] * scale`; a scale other than 1 needs a 32-bit output."""
    _on_device(tokens, table, out)
    _int_vector(tokens, "token ids")
    _require(out.shape == (tokens.shape[0], table.shape[1]), "output must be [tokens, width]")
    _require(scale == 1.0 or out.dtype == torch.float32, "scaled rows go into a 32-bit residual stream")
    if out.dtype == torch.float32 and (table.dtype != torch.float32 or scale != 1.0):   # rows widened into a 32-bit residual stream
        _require(table.is_contiguous() and out.is_contiguous(), "table and output must be contiguous")
        library = build.load_library("stream32.cu")
        return _check(library.tau_embedding_f32(_code(table), _pointer(tokens), _pointer(table), _pointer(out), ctypes.c_int(tokens.shape[0]),
                                                ctypes.c_int(table.shape[1]), ctypes.c_int(table.shape[0]), ctypes.c_float(scale), _stream()), "embedding")
    _require(table.dtype == out.dtype and table.is_contiguous() and out.is_contiguous(), "table and output must match")
    library = build.load_library("elementwise.cu")
    _check(library.tau_embedding(_code(table), _pointer(tokens), _pointer(table), _pointer(out), ctypes.c_int(tokens.shape[0]),
                                 ctypes.c_int(table.shape[1]), ctypes.c_int(table.shape[0]), _stream()), "embedding")


def rms_norm(values, weight, eps: float, out, rows=None, branch=None, groups: int = 1, branch_scale: float = 1.0) -> None:
    """`out[i] = norm(round(values[r] + branch[r])) * weight`, `r = rows[i]` or `i`; `values` is not changed.

    Where `values` is a 32-bit stream and the output is not, or there are two branches (a tuple), the sum is taken in
    32-bit (`values[r] + branch_scale * (a[r] + b[r])`) and only the output is rounded; a norm over `groups` > 1 pieces of the row,
    or a scale on the branches, needs the 32-bit stream as well."""
    if isinstance(branch, (tuple, list)) or values.dtype != out.dtype or groups != 1 or branch_scale != 1.0:
        return stream_add_norm(values, branch, weight, eps, out, rows=rows, update=False, groups=groups, branch_scale=branch_scale)
    _on_device(values, weight, out, rows, branch)
    width = values.shape[-1]
    _f32_vector(weight, width, "the norm weight")
    _require(values.is_contiguous() and out.is_contiguous() and out.dtype == values.dtype and out.shape[-1] == width,
             "norm input and output must be contiguous with the same dtype and width")
    if branch is not None:
        _require(branch.shape == values.shape and branch.dtype == values.dtype and branch.is_contiguous(), "branch must match the input")
    if rows is not None:
        _int_vector(rows, "row numbers")
    count = out.numel() // width
    _require(count == (rows.shape[0] if rows is not None else values.numel() // width), "output row count does not match")
    library = build.load_library("elementwise.cu")
    _check(library.tau_rms_norm(_code(values), _pointer(values), _pointer(branch), _pointer(rows), _pointer(weight), _pointer(out),
                                ctypes.c_int(count), ctypes.c_int(width), ctypes.c_float(eps), _stream()), "rms_norm")


def add_rms_norm(branch, residual, weight, eps: float, out, groups: int = 1, branch_scale: float = 1.0) -> None:
    """`residual = round(residual + branch)` in place; `out = norm(residual) * weight`.  A 32-bit residual beside an output
    of another dtype, two branches (a tuple), a norm in `groups` pieces or a scale on the branches go to `stream_add_norm`."""
    if isinstance(branch, (tuple, list)) or residual.dtype != out.dtype or groups != 1 or branch_scale != 1.0:
        return stream_add_norm(residual, branch, weight, eps, out, update=True, groups=groups, branch_scale=branch_scale)
    _on_device(branch, residual, weight, out)
    width = residual.shape[-1]
    _f32_vector(weight, width, "the norm weight")
    _require(branch.shape == residual.shape == out.shape and branch.dtype == residual.dtype == out.dtype,
             "branch, residual and output must match")
    _require(branch.is_contiguous() and residual.is_contiguous() and out.is_contiguous(), "tensors must be contiguous")
    library = build.load_library("elementwise.cu")
    _check(library.tau_add_rms_norm(_code(residual), _pointer(branch), _pointer(residual), _pointer(weight), _pointer(out),
                                    ctypes.c_int(residual.numel() // width), ctypes.c_int(width), ctypes.c_float(eps), _stream()),
           "add_rms_norm")


NORM_MAX_GROUPS = 1024


def stream_add_norm(stream, branches, weight, eps: float, out, rows=None, update: bool = True, groups: int = 1, branch_scale: float = 1.0) -> None:
    """A residual stream kept in 32-bit: `sum = stream[r] + branch_scale * (a[r] + b[r])` in 32-bit for up to two branches of any
    dtype (`branches`: None, a tensor or a tuple of one or two), `r = rows[i]` or `i`; with `update` (no `rows` then) the sum
    replaces `stream[r]`; `out[i] = sum / sqrt(mean(sum^2) + eps) * weight`, rounded once to the output's dtype.  With `groups` > 1
    the row is cut into that many equal consecutive pieces, each divided by its own root mean square."""
    _require(1 <= groups <= NORM_MAX_GROUPS and stream.shape[-1] % groups == 0, f"the groups (at most {NORM_MAX_GROUPS}) must divide the width")
    if branches is None:
        branches = ()
    elif not isinstance(branches, (tuple, list)):
        branches = (branches,)
    branches = tuple(branch for branch in branches if branch is not None)
    _require(len(branches) <= 2, "at most two branches join the stream at once")
    _on_device(stream, weight, out, rows, *branches)
    width = stream.shape[-1]
    _f32_vector(weight, width, "the norm weight")
    _require(stream.dtype == torch.float32 and stream.is_contiguous() and out.is_contiguous() and out.shape[-1] == width,
             "the stream must be contiguous float32 and the output as wide")
    for branch in branches:
        _require(branch.shape == stream.shape and branch.is_contiguous(), "a branch must match the stream")
    _require(not (update and rows is not None), "rows are gathered from a stream that is left as it is")
    if rows is not None:
        _int_vector(rows, "row numbers")
    count = out.numel() // width
    _require(count == (rows.shape[0] if rows is not None else stream.numel() // width), "output row count does not match")
    first = branches[0] if branches else None
    second = branches[1] if len(branches) > 1 else None
    library = build.load_library("stream32.cu")
    _check(library.tau_stream_add_norm(_code(out), _pointer(stream), _pointer(first), ctypes.c_int(_code(first) if first is not None else 0),
                                       _pointer(second), ctypes.c_int(_code(second) if second is not None else 0), _pointer(rows), _pointer(weight),
                                       _pointer(out), ctypes.c_int(count), ctypes.c_int(width), ctypes.c_float(eps), ctypes.c_int(1 if update else 0),
                                       ctypes.c_int(groups), ctypes.c_float(branch_scale), _stream()), "stream_add_norm")


def normed_pair_sum(left, right, left_weight, right_weight, eps: float, left_scale: float, right_scale: float, out) -> None:
    """`out = left_scale * left / rms(left) * left_weight + right_scale * right / rms(right) * right_weight`, each root mean square
    over the whole row (eps inside the root); everything float32 [rows, width]."""
    _on_device(left, right, left_weight, right_weight, out)
    rows, width = left.shape
    for tensor in (left, right, out):
        _require(tensor.dtype == torch.float32 and tensor.shape == (rows, width) and tensor.is_contiguous(), "both results and the output must be contiguous float32 [rows, width]")
    _f32_vector(left_weight, width, "the left weight")
    _f32_vector(right_weight, width, "the right weight")
    library = build.load_library("stream32.cu")
    _check(library.tau_normed_pair_sum(_pointer(left), _pointer(right), _pointer(left_weight), _pointer(right_weight), _pointer(out), ctypes.c_int(rows),
                                       ctypes.c_int(width), ctypes.c_float(eps), ctypes.c_float(left_scale), ctypes.c_float(right_scale), _stream()),
           "normed_pair_sum")


def gated_group_norm(values, weight, gate, out, groups: int, eps: float, normalize: bool, silu_gate: bool = False) -> None:
    """`values` [rows, width] in 32-bit; with `normalize` each of the `groups` equal parts of a row is divided by its root
    mean square (eps inside the root); then times `weight` (float32 [width] or None), times `sigmoid(gate)` or, with `silu_gate`,
    `gate * sigmoid(gate)` (the output's dtype, [rows, width], rows any distance apart, or None); rounded once to the output's
    dtype.  The output's rows may lie any distance apart too (a column range of a wider tensor)."""
    _on_device(values, weight, gate, out)
    rows, width = values.shape
    _require(values.dtype == torch.float32 and values.is_contiguous() and out.stride(1) == 1 and out.shape == values.shape,
             "values must be contiguous float32 and the output of the same shape")
    _require(groups > 0 and width % groups == 0, "the groups must divide the width")
    _f32_vector(weight, width, "the weight")
    if gate is not None:
        _require(gate.dtype == out.dtype and gate.shape == values.shape and gate.stride(1) == 1, "the gate must have the output's dtype and shape")
    library = build.load_library("stream32.cu")
    _check(library.tau_gated_group_norm(_code(out), _pointer(values), _pointer(weight), _pointer(gate),
                                        ctypes.c_longlong(0 if gate is None else gate.stride(0)), _pointer(out), ctypes.c_longlong(out.stride(0)), ctypes.c_int(rows),
                                        ctypes.c_int(groups), ctypes.c_int(width // groups), ctypes.c_float(eps), ctypes.c_int(1 if normalize else 0),
                                        ctypes.c_int(1 if silu_gate else 0), _stream()), "gated_group_norm")


def silu_mul(stacked, out, relu: bool = False) -> None:
    """`out[r, c] = silu(stacked[r, c]) * stacked[r, width + c]`; with `relu` the activation is `max(z, 0)` instead."""
    _on_device(stacked, out)
    width = out.shape[-1]
    _require(stacked.shape[-1] == 2 * width and stacked.shape[0] == out.shape[0] and stacked.dtype == out.dtype,
             "input must be [rows, 2 * width] and output [rows, width]")
    _require(stacked.is_contiguous() and out.is_contiguous(), "tensors must be contiguous")
    library = build.load_library("elementwise.cu")
    _check(library.tau_silu_mul(_code(out), _pointer(stacked), _pointer(out), ctypes.c_longlong(out.shape[0]), ctypes.c_int(width),
                                ctypes.c_int(1 if relu else 0), _stream()), "silu_mul")


# ---------------------------------------------------------------------------- products
def gemm_simt(values, weight, bias, out) -> None:
    """`out = values @ weight.T + bias` on the 32-bit pipes; any sizes."""
    _on_device(values, weight, bias, out)
    rows, depth = values.shape
    features = weight.shape[0]
    _require(weight.shape[1] == depth and out.shape == (rows, features), "shapes must be [M,K] x [N,K] -> [M,N]")
    _require(values.dtype == weight.dtype, "input and weight must have the same dtype")
    _require(out.dtype == values.dtype or out.dtype == torch.float32, "output must have the input's dtype or float32")
    _f32_vector(bias, features, "the bias")
    library = build.load_library("gemm_simt.cu")
    _check(library.tau_gemm_simt(_code(values), _code(out), _pointer(values), _pointer(weight), _pointer(bias), _pointer(out),
                                 ctypes.c_int(rows), ctypes.c_int(features), ctypes.c_int(depth),
                                 ctypes.c_longlong(values.stride(0)), ctypes.c_longlong(weight.stride(0)),
                                 ctypes.c_longlong(out.stride(0)), _stream()), "gemm_simt")


def gemm_simt_batched(values, weight, out) -> None:
    """`out[:, b] = values[:, b] @ weight[b].T` for every `b` in one launch, on the 32-bit pipes: `values` [M, B, K],
    `weight` [B, N, K], `out` [M, B, N]; the three may be views whose rows and batches lie any distance apart."""
    _on_device(values, weight, out)
    rows, batch, depth = values.shape
    features = weight.shape[1]
    _require(weight.shape == (batch, features, depth) and out.shape == (rows, batch, features), "shapes must be [M,B,K] x [B,N,K] -> [M,B,N]")
    _require(values.dtype == weight.dtype and out.dtype in (values.dtype, torch.float32), "input and weight must have the same dtype")
    library = build.load_library("gemm_simt.cu")
    _check(library.tau_gemm_simt_batched(_code(values), _code(out), _pointer(values), _pointer(weight), _pointer(out), ctypes.c_int(rows),
                                         ctypes.c_int(features), ctypes.c_int(depth), ctypes.c_longlong(values.stride(0)),
                                         ctypes.c_longlong(weight.stride(1)), ctypes.c_longlong(out.stride(0)), ctypes.c_int(batch),
                                         ctypes.c_longlong(values.stride(1)), ctypes.c_longlong(weight.stride(0)), ctypes.c_longlong(out.stride(1)),
                                         _stream()), "gemm_simt_batched")


SKINNY_MAX_ROWS = 32      # what the skinny kernel accepts
SKINNY_BEST_ROWS = 8      # up to here it beats the tcgen05 product cut along K (Qwen3-8B layer shapes: 72 us against 81 us per
                          # layer at 8 rows, 97 against 82 at 12, 152 against 91 at 32)
SKINNY_SMALL_ROWS = 16    # ... and up to here where the weight is small: the tcgen05 kernel's set-up (tensor memory, barriers,
SKINNY_SMALL_WEIGHT = 8 << 20   # tensor maps, the meeting of its K ranges) costs about 6 us whatever the size, the skinny kernel's
                          # about 2.5 us.  Qwen3-0.6B layer shapes (2 to 6 M elements per weight): 18.7 us against 24.4 us per layer
                          # at 16 rows, 26.0 against 25.9 at 24.  Qwen3-8B shapes (17 to 100 M): 101 against 80 us at 16 rows.


def _skinny_wins(values, weight) -> bool:
    rows = values.shape[0]
    return rows <= SKINNY_BEST_ROWS or (rows <= SKINNY_SMALL_ROWS and weight.numel() <= SKINNY_SMALL_WEIGHT)


def _skinny_fits(values, weight, out) -> bool:
    return (values.dtype == torch.bfloat16 and values.shape[0] <= SKINNY_MAX_ROWS and values.shape[1] % 8 == 0
            and values.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and values.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0)


def gemm_skinny(values, weight, bias, out, gated: bool = False) -> None:
    """bfloat16 product for at most 32 activation rows, bound by streaming `weight` once.

    `gated`: the weight's rows are groups of 8 gate rows and their 8 up rows; `out` is `[M, N / 2]` = silu(gate) * up.
    """
    _on_device(values, weight, bias, out)
    rows, depth = values.shape
    features = weight.shape[0]
    _require(weight.shape[1] == depth and out.shape == (rows, features // 2 if gated else features), "shapes must be [M,K] x [N,K] -> [M,N]")
    _require(not gated or features % 16 == 0, "a gated product needs a multiple of 16 weight rows")
    _require(values.dtype == weight.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32),
             "inputs must be bfloat16 and the output bfloat16 or float32")
    _require(_skinny_fits(values, weight, out), "needs M <= 32, K % 8 == 0 and 16-byte aligned rows")
    _f32_vector(bias, features, "the bias")
    library = build.load_library("gemm_skinny.cu")
    _check(library.tau_gemm_skinny(_code(out), _pointer(values), _pointer(weight), _pointer(bias), _pointer(out), ctypes.c_int(rows),
                                   ctypes.c_int(features), ctypes.c_int(depth), ctypes.c_longlong(values.stride(0)),
                                   ctypes.c_longlong(weight.stride(0)), ctypes.c_longlong(out.stride(0)), ctypes.c_int(1 if gated else 0),
                                   _stream()), "gemm_skinny")


def _tc_fits(values, weight, out) -> bool:
    return (values.dtype == torch.bfloat16 and values.shape[1] % 8 == 0 and values.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
            and values.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (of the current one if none is named; 148, a B200's, where there is no GPU
    to ask, which only the host-side tests of the rules below meet)."""
    if not torch.cuda.is_available():
        return 148
    index = torch.cuda.current_device() if device is None or torch.device(device).index is None else torch.device(device).index
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


_tc_workspace = {}
_TC_TICKETS = 4096


def _tc_workspace_for(device):
    """The partial tiles and tickets of a product cut along K; one pair per device and stream order.
    A 128 x 128 float partial for each of two blocks per SM (19.4 MB on 148 SMs)."""
    entry = _tc_workspace.get(device)
    if entry is None:
        entry = _tc_workspace[device] = (torch.empty(2 * sm_count(device) * 128 * 128, dtype=torch.float32, device=device),
                                         torch.zeros(_TC_TICKETS, dtype=torch.int32, device=device))   # zero once; the kernel leaves them at zero
    return entry


def gemm_tc(values, weight, bias, out, token_box: int = 0, gated: bool = False, splits: int = 0, pair: int = -1, cluster: bool = True) -> None:
    """bfloat16 product on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory); any M and N, K % 8 == 0.

    `gated`: the weight's rows are groups of 8 gate rows and their 8 up rows; `out` is `[M, N / 2]` = silu(gate) * up.
    `splits`: K ranges that the product is cut into (0: chosen from the sizes, for products with few tiles).
    `cluster`: False makes the K ranges of a tile meet in a workspace in global memory even where they could meet in the
    shared memory of a thread-block cluster.
    `pair`: 256 x 256 tiles on pairs of SMs (tcgen05 `cta_group::2`) where the 256-token tile is used: -1 yes, 0 no, 1 insist.
    """
    _on_device(values, weight, bias, out)
    rows, depth = values.shape
    features = weight.shape[0]
    _require(weight.shape[1] == depth and out.shape == (rows, features // 2 if gated else features), "shapes must be [M,K] x [N,K] -> [M,N]")
    _require(not gated or (features % 16 == 0 and out.dtype == torch.bfloat16), "a gated product needs a multiple of 16 weight rows and a bfloat16 output")
    _require(values.dtype == weight.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32),
             "inputs must be bfloat16 and the output bfloat16 or float32")
    _require(_tc_fits(values, weight, out), "needs K % 8 == 0 and 16-byte aligned rows")
    _f32_vector(bias, features, "the bias")
    library = build.load_library("gemm_tc.cu")
    workspace, tickets = _tc_workspace_for(out.device)
    _check(library.tau_gemm_tc(_code(out), _pointer(values), _pointer(weight), _pointer(bias), _pointer(out), ctypes.c_int(rows),
                               ctypes.c_int(features), ctypes.c_int(depth), ctypes.c_longlong(values.stride(0)),
                               ctypes.c_longlong(weight.stride(0)), ctypes.c_longlong(out.stride(0)), ctypes.c_int(token_box),
                               ctypes.c_int(1 if gated else 0), ctypes.c_int(splits), _pointer(workspace),
                               ctypes.c_longlong(workspace.numel()), _pointer(tickets), ctypes.c_int(pair), ctypes.c_int(1 if cluster else 0), _stream()), "gemm_tc")


def gemm_tc_groups(values, weights, out, bounds, gated: bool = False) -> None:
    """One tensor-core product per group of consecutive rows: rows `bounds[g] .. bounds[g + 1]` of `values` [M, K] meet
    `weights[g]` ([groups, N, K]) and land in the same rows of `out` ([M, N], or [M, N / 2] = silu(gate) * up with `gated`).
    `bounds` is a host list of `groups + 1` ascending row numbers.  bfloat16, K % 8 == 0, 16-byte aligned rows."""
    _on_device(values, weights, out)
    rows, depth = values.shape
    groups, features = weights.shape[0], weights.shape[1]
    _require(weights.shape[2] == depth and weights.is_contiguous() and out.shape == (rows, features // 2 if gated else features),
             "shapes must be [M,K] x [G,N,K] -> [M,N]")
    _require(len(bounds) == groups + 1 and bounds[0] == 0 and bounds[-1] <= rows, "bounds must start at 0 and end within the rows")
    _require(values.dtype == weights.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32) and (not gated or out.dtype == torch.bfloat16),
             "inputs must be bfloat16 and the output bfloat16 or float32 (bfloat16 for a gated product)")
    _require(_tc_fits(values, weights[0], out) and (not gated or features % 16 == 0), "needs K % 8 == 0 and 16-byte aligned rows")
    library = build.load_library("gemm_tc.cu")
    workspace, tickets = _tc_workspace_for(out.device)
    table = (ctypes.c_int * (groups + 1))(*bounds)
    launched = sum(1 for index in range(groups) if bounds[index + 1] > bounds[index])
    _check(library.tau_gemm_tc_groups(_code(out), _pointer(values), _pointer(weights), _pointer(out), table, ctypes.c_int(groups), ctypes.c_int(features),
                                      ctypes.c_int(depth), ctypes.c_longlong(values.stride(0)), ctypes.c_longlong(weights.stride(1)),
                                      ctypes.c_longlong(out.stride(0)), ctypes.c_longlong(weights.stride(0)), ctypes.c_int(1 if gated else 0),
                                      _pointer(workspace), ctypes.c_longlong(workspace.numel()), _pointer(tickets), _stream()), "gemm_tc_groups", launched)


def gemm_tc_status() -> int:
    """0 unless a bounded wait inside the tensor-core product ran out (synchronises the device)."""
    return build.load_library("gemm_tc.cu").tau_gemm_tc_status()


GATE_GROUP = 8   # rows of a gate (and of its up) that lie together in a weight prepared for `linear_gated`


_prefer_optimized = True


def prefer_optimized(enabled: bool) -> None:
    """`--optimize-kernel true|false` (crates/server/src/args.rs: "Prefer optimized kernels ... false: use reference
    kernels").  With `False` every product is the plain tiled kernel, every attention the one-warp-per-head kernel over
    the pages, and nothing is fused: the slow kernels that the others are checked against, for telling a kernel's
    fault from the engine's.  Set it before the model is built: a feed-forward decides then whether its gate and up
    rows are interleaved for the gated product."""
    global _prefer_optimized
    _prefer_optimized = bool(enabled)


def optimized_preferred() -> bool:
    return _prefer_optimized


def gated_fits(in_features: int, out_features: int, dtype) -> bool:
    """Whether `linear_gated` serves a gate/up pair of these sizes (else: `linear`, then `silu_mul`)."""
    return _prefer_optimized and dtype == torch.bfloat16 and in_features % 8 == 0 and out_features % GATE_GROUP == 0


def linear_gated(values, weight, out) -> None:
    """`out = silu(values @ gate.T) * (values @ up.T)` in one product; `weight` holds groups of 8 gate rows followed by
    their 8 up rows (see `parts.linear.StackedLinear(interleave=...)`)."""
    if _skinny_fits(values, weight, out) and _skinny_wins(values, weight):
        return gemm_skinny(values, weight, None, out, gated=True)
    _require(_tc_fits(values, weight, out), "the gated product needs bfloat16, K % 8 == 0 and 16-byte aligned rows")
    gemm_tc(values, weight, None, out, gated=True)


def linear(values, weight, bias, out) -> None:
    """`out = values @ weight.T + bias` with the kernel that fits the dtype and the sizes."""
    if values.dtype == torch.bfloat16 and _prefer_optimized:
        if _skinny_fits(values, weight, out) and _skinny_wins(values, weight):
            return gemm_skinny(values, weight, bias, out)
        if _tc_fits(values, weight, out):
            return gemm_tc(values, weight, bias, out)
    gemm_simt(values, weight, bias, out)


# ---------------------------------------------------------------------------- attention
def attention_prepare(projected, queries, keys, values, write_cache: bool, q_weight, k_weight, eps: float, cos, sin,
                      rotary_dim: int, positions, token_seq, page_rows, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
    """Per-head norm and rotation of the projected queries and keys; keys and values go to their cache pages.

    `projected` is `[tokens, (n_heads + 2 n_kv_heads) head_dim]` (only the query part is
    needed when `write_cache` is false); `queries` receives `[tokens, n_heads head_dim]`.
    """
    _on_device(projected, queries, keys, values, q_weight, k_weight, cos, sin, positions, token_seq, page_rows)
    tokens = projected.shape[0]
    needed = (n_heads + (2 * n_kv_heads if write_cache else 0)) * head_dim
    _require(projected.shape[1] >= needed, f"projected rows must hold {needed} elements")
    _require(queries.shape == (tokens, n_heads * head_dim) and queries.is_contiguous() and queries.dtype == projected.dtype,
             "queries must be [tokens, n_heads * head_dim]")
    _require(head_dim % 16 == 0 and 16 <= head_dim <= 256, "head_dim must be a multiple of 16 between 16 and 256")
    _require(keys.dtype == projected.dtype and values.dtype == projected.dtype, "cache dtype must match the activations")
    _require(keys.shape[1:] == (n_kv_heads, PAGE_TOKENS, head_dim) and keys.is_contiguous() and values.is_contiguous()
             and values.shape == keys.shape, "cache pages must be [pages, n_kv_heads, 64, head_dim]")
    _f32_vector(q_weight, head_dim, "the q norm weight")
    _f32_vector(k_weight, head_dim, "the k norm weight")
    if rotary_dim:
        _require(cos is not None and sin is not None and cos.dtype == torch.float32 and cos.shape == sin.shape
                 and cos.shape[1] == rotary_dim // 2 and cos.is_contiguous() and sin.is_contiguous(),
                 "rotation tables must be float32 [positions, rotary_dim / 2]")
    _int_vector(positions, "positions")
    _int_vector(token_seq, "token_seq")
    _require(page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous(), "page rows must be int32 [sequences, stride]")
    library = build.load_library("attention_generic.cu")
    _check(library.tau_attention_prepare(
        _code(projected), _pointer(projected), ctypes.c_longlong(projected.stride(0)), _pointer(queries), _pointer(keys), _pointer(values),
        _pointer(q_weight), _pointer(k_weight), ctypes.c_float(eps), _pointer(cos), _pointer(sin), ctypes.c_int(rotary_dim),
        _pointer(positions), _pointer(token_seq), _pointer(page_rows), ctypes.c_int(page_rows.shape[1]), ctypes.c_int(PAGE_TOKENS),
        ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim), ctypes.c_int(1 if write_cache else 0),
        _stream()), "attention_prepare")


def attention_generic(queries, keys, values, out, positions, token_seq, page_rows, n_heads: int, n_kv_heads: int, head_dim: int,
                      scale: float, window: int) -> None:
    _on_device(queries, keys, values, out, positions, token_seq, page_rows)
    tokens = queries.shape[0]
    _require(queries.shape == (tokens, n_heads * head_dim) and out.shape == queries.shape and queries.is_contiguous() and out.is_contiguous()
             and out.dtype == queries.dtype == keys.dtype == values.dtype, "queries and output must be [tokens, n_heads * head_dim]")
    _require(head_dim % 16 == 0 and 16 <= head_dim <= 256, "head_dim must be a multiple of 16 between 16 and 256")
    _require(n_heads % n_kv_heads == 0, "n_heads must be a multiple of n_kv_heads")
    _require(keys.shape[1:] == (n_kv_heads, PAGE_TOKENS, head_dim) and keys.is_contiguous() and values.is_contiguous()
             and values.shape == keys.shape, "cache pages must be [pages, n_kv_heads, 64, head_dim]")
    _require(page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous(), "page rows must be int32 [sequences, stride]")
    library = build.load_library("attention_generic.cu")
    _check(library.tau_attention_generic(
        _code(queries), _pointer(queries), _pointer(keys), _pointer(values), _pointer(out), _pointer(positions), _pointer(token_seq),
        _pointer(page_rows), ctypes.c_int(page_rows.shape[1]), ctypes.c_int(PAGE_TOKENS), ctypes.c_int(tokens), ctypes.c_int(n_heads),
        ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim), ctypes.c_float(scale), ctypes.c_int(window), _stream()), "attention")


def decode_splits(n_seqs: int, max_len: int, kv_blocks: int = 8, sms: Optional[int] = None) -> int:
    """Number of context splits that decode attention uses for this many sequences of at most this length.

    `kv_blocks` is the number of blocks per sequence and split (KV heads times head passes).  Four blocks of the
    decode kernel fit an SM, so the aim is the largest number of splits whose blocks are all resident at once
    (one wave: a second, partly filled wave costs more than the extra parallelism gives), each split at least 64
    positions long.  Up to 16 splits merge inside a thread-block cluster, through shared memory, which saves 2 to 5 us
    against the meeting in global memory (one sequence of 2,049 positions: 9.3 us with 16 splits in a cluster, 12.0 us
    with 16 that meet in global memory; 8 sequences: 17.8 against 20.4 us with 8 splits).  Clusters of more than 8 blocks
    are placed badly once they fill more than half of the SMs' places (4 sequences, 16 splits: 19.5 us against 14.1 us
    with 8), so then 8 are used.  Beyond 8,192 positions up to 32 splits meet in global memory (one sequence of 32,001
    positions: 40.4 us with 32, 54.9 us with 16 in a cluster).  The length is rounded up to a power of two first, so
    that a captured graph (whose key holds this number) serves a whole range of lengths.
    """
    sms = sms or sm_count()
    bucket = 1 << max(0, (max_len - 1).bit_length())
    blocks = max(1, n_seqs * kv_blocks)
    splits = max(1, min(4 * sms // blocks, bucket // 64, 16 if bucket <= 8192 else 32))
    if 8 < splits <= 16 and blocks * splits > 2 * sms:
        splits = 8
    # The splits of a (sequence, KV head) are one cluster, and clusters do not fill the last places of the machine: on 148 SMs
    # (592 places) 576 blocks in clusters of 3, 6 or 8 and 560 in clusters of 7 took a second wave (9 sequences of 2,048
    # positions: 31.1 us with 8 splits, 21.2 us with 7; 24 sequences: 59.6 us with 3, 44.6 us with 2), while 560 in clusters of 5
    # and 512 in clusters of 8 and 576 in pairs were resident at once.  So pairs may fill 98% of the places, clusters of up to 5
    # 95%, larger ones 87%.
    while 1 < splits <= 16 and blocks * splits * 100 > 4 * sms * _CLUSTER_FILL[min(splits, 6)]:
        splits -= 1
    return splits


_CLUSTER_FILL = {2: 98, 3: 95, 4: 95, 5: 95, 6: 87}   # per cent of the machine's places that clusters of this size (6: and more) fill


_decode_scratch = {}
_decode_tickets = {}


def attention_decode(queries, keys, values, out, seq_len, page_rows, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                     window: int, splits: int, prepare=None, cluster_merge: bool = True) -> None:
    """One query token per sequence (its last position) over `seq_len` cached positions, split along the context.

    `prepare` (bfloat16 only) is `(projected, q_weight, k_weight, eps, cos, sin, rotary_dim, write_cache)`: the kernel
    then takes queries, the newest key and the newest value from the stacked projection itself (per-head norm,
    rotation, cache write), `queries` may be None, and no prepare kernel is needed before it.
    `cluster_merge` (bfloat16): up to 16 splits are one thread-block cluster and merge through shared memory; False makes
    them meet in global memory like larger numbers of splits.
    """
    _on_device(queries, keys, values, out, seq_len, page_rows)
    n_seqs = out.shape[0]
    _require(out.shape == (n_seqs, n_heads * head_dim) and out.is_contiguous() and out.dtype == keys.dtype == values.dtype,
             "output must be [sequences, n_heads * head_dim] in the cache's dtype")
    if queries is not None:
        _require(queries.shape == out.shape and queries.is_contiguous() and queries.dtype == out.dtype, "queries must match the output")
    _require(head_dim % 16 == 0 and 16 <= head_dim <= 256, "head_dim must be a multiple of 16 between 16 and 256")
    _require(n_heads % n_kv_heads == 0, "n_heads must be a multiple of n_kv_heads")
    _require(keys.shape[1:] == (n_kv_heads, PAGE_TOKENS, head_dim) and keys.is_contiguous() and values.is_contiguous()
             and values.shape == keys.shape, "cache pages must be [pages, n_kv_heads, 64, head_dim]")
    _int_vector(seq_len, "sequence lengths")
    _require(seq_len.numel() == n_seqs and page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous()
             and page_rows.shape[0] == n_seqs, "one length and one row of pages per sequence")
    _require(1 <= splits <= 256 and (out.dtype != torch.bfloat16 or splits <= 2 * head_dim), "splits must lie between 1 and 256 (and 2 * head_dim in bfloat16)")
    projected = q_weight = k_weight = cos = sin = None
    eps, rotary_dim, write_cache = 0.0, 0, False
    if prepare is not None:
        projected, q_weight, k_weight, eps, cos, sin, rotary_dim, write_cache = prepare
        _on_device(projected, q_weight, k_weight, cos, sin)
        _require(out.dtype == torch.bfloat16 and projected.dtype == torch.bfloat16, "the fused form is bfloat16 only")
        needed = (n_heads + (2 * n_kv_heads if write_cache else 0)) * head_dim
        _require(projected.shape[0] == n_seqs and projected.shape[1] >= needed and projected.stride(1) == 1,
                 f"projected rows must hold {needed} elements")
        _f32_vector(q_weight, head_dim, "the q norm weight")
        _f32_vector(k_weight, head_dim, "the k norm weight")
        if rotary_dim:
            _require(cos is not None and sin is not None and cos.dtype == torch.float32 and cos.shape == sin.shape
                     and cos.shape[1] == rotary_dim // 2 and cos.is_contiguous() and sin.is_contiguous(),
                     "rotation tables must be float32 [positions, rotary_dim / 2]")
    else:
        _require(queries is not None, "queries are needed unless the kernel prepares them")
    library = build.load_library("attention_decode.cu", (f"TAU_HEAD_DIM={head_dim}", f"TAU_DTYPE={_code(out)}"))
    library.tau_attention_decode_scratch.restype = ctypes.c_longlong
    library.tau_attention_decode_tickets.restype = ctypes.c_longlong
    floats = library.tau_attention_decode_scratch(ctypes.c_int(n_seqs), ctypes.c_int(n_heads), ctypes.c_int(splits))
    scratch = tickets = None
    if floats:
        key = (out.device, _stream_handle())
        scratch = _decode_scratch.get(key)
        if scratch is None or scratch.numel() < floats:
            scratch = _decode_scratch[key] = torch.empty(floats, dtype=torch.float32, device=out.device)
        if out.dtype == torch.bfloat16:
            wanted = library.tau_attention_decode_tickets(ctypes.c_int(n_seqs), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads))
            tickets = _decode_tickets.get(key)
            if tickets is None or tickets.numel() < wanted:   # zero once; the kernel leaves them at zero
                tickets = _decode_tickets[key] = torch.zeros(max(wanted, 1024), dtype=torch.int32, device=out.device)
    launches = 1 if (splits == 1 or out.dtype == torch.bfloat16) else 2
    _check(library.tau_attention_decode(
        _pointer(queries), _pointer(keys), _pointer(values), _pointer(out), _pointer(seq_len), _pointer(page_rows),
        ctypes.c_int(page_rows.shape[1]), ctypes.c_int(PAGE_TOKENS), ctypes.c_int(n_seqs), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads),
        ctypes.c_float(scale), ctypes.c_int(window), ctypes.c_int(splits), _pointer(scratch),
        ctypes.c_longlong(0 if scratch is None else scratch.numel()), _pointer(tickets),
        _pointer(projected), ctypes.c_longlong(0 if projected is None else projected.stride(0)), _pointer(q_weight), _pointer(k_weight),
        ctypes.c_float(eps), _pointer(cos), _pointer(sin), ctypes.c_int(rotary_dim), ctypes.c_int(1 if write_cache else 0),
        ctypes.c_int(1 if cluster_merge else 0), _stream()),
        "attention_decode", launches)


def attention_decode_fused(projected, keys, values, out, step, page_rows, write_cache: bool, q_weight, k_weight, eps: float, cos, sin,
                           rotary_dim: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int) -> bool:
    """Prepare and decode attention in one kernel, where that exists: every sequence brings one token and the dtype is
    bfloat16.  Returns False (and does nothing) otherwise; the caller then runs `attention_prepare` and `attention`."""
    if not (step.all_single and projected.dtype == torch.bfloat16 and _prefer_optimized):
        return False
    splits = min(step.decode_splits or decode_splits(step.n_seqs, step.max_len), 2 * head_dim)   # the kernel's limit on a given number
    attention_decode(None, keys, values, out, step.seq_len, page_rows, n_heads, n_kv_heads, head_dim, scale, window, splits,
                     prepare=(projected, q_weight, k_weight, eps, cos, sin, rotary_dim, write_cache))
    return True


def attention_prefill(queries, keys, values, out, cu_seqlens, seq_start, page_rows, n_heads: int, n_kv_heads: int, head_dim: int,
                      scale: float, window: int, sinks=None) -> None:
    """bfloat16 causal attention of runs of new tokens (`cu_seqlens` bounds them, `seq_start` positions were cached before).
    `sinks` (float32 [n_heads] or None): `exp(sink)` joins each head's softmax denominator."""
    _on_device(queries, keys, values, out, cu_seqlens, seq_start, page_rows, sinks)
    _f32_vector(sinks, n_heads, "the sinks")
    tokens = queries.shape[0]
    n_seqs = seq_start.numel()
    _require(queries.dtype == torch.bfloat16 == out.dtype == keys.dtype == values.dtype, "the tensor-core prefill kernel is bfloat16 only")
    _require(queries.shape == (tokens, n_heads * head_dim) and out.shape == queries.shape and queries.is_contiguous() and out.is_contiguous(),
             "queries and output must be [tokens, n_heads * head_dim]")
    _require(head_dim % 16 == 0 and 16 <= head_dim <= 256, "head_dim must be a multiple of 16 between 16 and 256")
    _require(n_heads % n_kv_heads == 0, "n_heads must be a multiple of n_kv_heads")
    _require(keys.shape[1:] == (n_kv_heads, PAGE_TOKENS, head_dim) and keys.is_contiguous() and values.is_contiguous()
             and values.shape == keys.shape, "cache pages must be [pages, n_kv_heads, 64, head_dim]")
    _int_vector(cu_seqlens, "cu_seqlens")
    _int_vector(seq_start, "seq_start")
    _require(cu_seqlens.numel() == n_seqs + 1 and page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous()
             and page_rows.shape[0] == n_seqs, "one run and one row of pages per sequence")
    library = build.load_library("attention_prefill.cu", (f"TAU_HEAD_DIM={head_dim}",))
    _check(library.tau_attention_prefill(
        _pointer(queries), _pointer(keys), _pointer(values), _pointer(out), _pointer(cu_seqlens), _pointer(seq_start), _pointer(page_rows),
        ctypes.c_int(page_rows.shape[1]), ctypes.c_int(PAGE_TOKENS), ctypes.c_int(n_seqs), ctypes.c_int(tokens), ctypes.c_int(n_heads),
        ctypes.c_int(n_kv_heads), ctypes.c_float(scale), ctypes.c_int(window), _pointer(sinks), _stream()), "attention_prefill")


_prefill_schedule = {}   # (device, stream) -> the two counters by which the blocks of the tensor-core prefill kernel share out its tiles


def attention_prefill_tc(queries, keys, values, out, cu_seqlens, seq_start, page_rows, n_heads: int, n_kv_heads: int, head_dim: int,
                         scale: float, window: int, chunk: int = 0, sink: bool = False, out_scale: float = 1.0, distance=None, sigmoid_weights: bool = False,
                         head_offset=None, head_gate=None) -> None:
    """The same as `attention_prefill` on the tcgen05 tensor cores (accumulators in tensor memory); head sizes 64 and 128.
    Beyond it: with `chunk` a query sees only the keys of its own chunk of `chunk` positions (counted from position 0 of the
    sequence) instead of a window; with `sink` the softmax's denominator has one added; the result is multiplied by `out_scale`;
    `out` may be a column range of a wider tensor whose rows start on 16-byte borders.  `distance` (float32 [n_heads, 2] = (r1, r2)):
    `r1 * ln(1 + r2 * (i - j))` is taken off the score of key j for the query at i.  `sigmoid_weights`: every visible key weighs
    `sigmoid(score + head_offset[head])` (float32 [n_heads] or None) instead of its share of a softmax.  `head_gate` (bfloat16
    [tokens, n_heads], rows any distance apart): a head's result is multiplied by the sigmoid of its number."""
    _on_device(queries, keys, values, out, cu_seqlens, seq_start, page_rows, distance, head_offset, head_gate)
    if distance is not None:
        _require(distance.dtype == torch.float32 and distance.shape == (n_heads, 2) and distance.is_contiguous(), "the distance numbers must be float32 [heads, 2]")
    _f32_vector(head_offset, n_heads, "the heads' offsets")
    _require(not (sigmoid_weights and sink), "sigmoid weights have no denominator for a sink to join")
    if head_gate is not None:
        _require(head_gate.dtype == torch.bfloat16 and head_gate.shape == (queries.shape[0], n_heads) and head_gate.stride(1) == 1, "the gate must be bfloat16 [tokens, heads]")
    tokens = queries.shape[0]
    n_seqs = seq_start.numel()
    _require(head_dim in (64, 128), "the tensor-core prefill kernel serves head sizes 64 and 128")
    _require(queries.dtype == torch.bfloat16 == out.dtype == keys.dtype == values.dtype, "the tensor-core prefill kernel is bfloat16 only")
    _require(queries.shape == (tokens, n_heads * head_dim) and out.shape == queries.shape and queries.is_contiguous() and out.stride(1) == 1
             and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0, "queries and output must be [tokens, n_heads * head_dim], output rows on 16-byte borders")
    _require(n_heads % n_kv_heads == 0, "n_heads must be a multiple of n_kv_heads")
    _require(keys.shape[1:] == (n_kv_heads, PAGE_TOKENS, head_dim) and keys.is_contiguous() and values.is_contiguous()
             and values.shape == keys.shape, "cache pages must be [pages, n_kv_heads, 64, head_dim]")
    _require(not (window and chunk), "a window or a chunk, not both")
    _int_vector(cu_seqlens, "cu_seqlens")
    _int_vector(seq_start, "seq_start")
    _require(cu_seqlens.numel() == n_seqs + 1 and page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous()
             and page_rows.shape[0] == n_seqs, "one run and one row of pages per sequence")
    library = build.load_library("attention_prefill_tc.cu", (f"TAU_HEAD_DIM={head_dim}",))
    key = (out.device, _stream_handle())
    schedule = _prefill_schedule.get(key)
    if schedule is None:   # zero once; the kernel leaves it at zero
        schedule = _prefill_schedule[key] = torch.zeros(2, dtype=torch.int32, device=out.device)
    _check(library.tau_attention_prefill_tc(
        _pointer(queries), _pointer(keys), _pointer(values), _pointer(out), _pointer(cu_seqlens), _pointer(seq_start), _pointer(page_rows),
        ctypes.c_int(page_rows.shape[1]), ctypes.c_int(PAGE_TOKENS), ctypes.c_longlong(keys.shape[0]), ctypes.c_int(n_seqs),
        ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_float(scale), ctypes.c_int(window), ctypes.c_int(chunk),
        ctypes.c_int(1 if sink else 0), ctypes.c_float(out_scale), ctypes.c_longlong(out.stride(0)), _pointer(schedule), _pointer(distance),
        ctypes.c_int(1 if sigmoid_weights else 0), _pointer(head_offset), _pointer(head_gate), ctypes.c_longlong(0 if head_gate is None else head_gate.stride(0)),
        _stream()), "attention_prefill_tc")


def attention_prefill_tc_status(head_dim: int) -> int:
    """0 unless a bounded wait inside the tensor-core prefill kernel ran out (synchronises the device)."""
    return build.load_library("attention_prefill_tc.cu", (f"TAU_HEAD_DIM={head_dim}",)).tau_attention_prefill_tc_status()


def attention(queries, keys, values, out, step, page_rows, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
              window: int) -> None:
    """Causal attention of the step's tokens over their sequences' cache pages (which hold the step's own keys already)."""
    if not _prefer_optimized:
        return attention_generic(queries, keys, values, out, step.positions, step.token_seq, page_rows, n_heads, n_kv_heads, head_dim, scale, window)
    if step.all_single:
        splits = min(step.decode_splits or decode_splits(step.n_seqs, step.max_len), 2 * head_dim)
        return attention_decode(queries, keys, values, out, step.seq_len, page_rows, n_heads, n_kv_heads, head_dim, scale, window, splits)
    if queries.dtype == torch.bfloat16:
        # The tensor-memory kernel addresses the cache by 32-bit rows (pages x kv heads x 64); a larger cache goes to the other kernel.
        rows_fit = keys.shape[0] * n_kv_heads * PAGE_TOKENS <= 0x7FFFFFFF
        prefill = attention_prefill_tc if head_dim in (64, 128) and rows_fit else attention_prefill
        return prefill(queries, keys, values, out, step.cu_seqlens, step.seq_start, page_rows, n_heads, n_kv_heads, head_dim, scale, window)
    attention_generic(queries, keys, values, out, step.positions, step.token_seq, page_rows, n_heads, n_kv_heads, head_dim, scale, window)


# ---------------------------------------------------------------------------- latent attention
def latent_prepare(down, latent_weight, eps: float, q, queries, rows, inv_freq, rotary_dim: int, positions, token_seq, page_rows,
                   n_heads: int, head_dim: int, rot_dim: int, rank: int, write_rows: bool = True, latent_out=None) -> None:
    """`down` [tokens, rank + rot_dim]: its first `rank` elements, RMS-normed with `latent_weight`, and its last `rot_dim`,
    rotated, go to the token's row of the cache pages `rows` [pages, 64, rank + rot_dim].  `q` [tokens, n_heads *
    (head_dim + rot_dim)]: each head's last `rot_dim` elements, rotated, go to `queries[token, head, rank:]`
    (`queries` [tokens, n_heads, rank + rot_dim]; its first `rank` elements per head are another kernel's to fill).
    The rotation turns the pair (2i, 2i + 1), i < rotary_dim / 2, by `position * inv_freq[i]`.  `queries` may be None (no query
    is prepared); `latent_out` [tokens, rank] receives the normalised latents side by side as well."""
    _on_device(down, latent_weight, q, queries, rows, inv_freq, positions, token_seq, page_rows, latent_out)
    tokens, width = q.shape[0], rank + rot_dim
    _require(q.shape[1] == n_heads * (head_dim + rot_dim), "q must be [tokens, n_heads * (head_dim + rot_dim)]")
    if queries is not None:
        _require(queries.shape == (tokens, n_heads, width) and queries.is_contiguous() and queries.dtype == q.dtype,
                 "queries must be [tokens, n_heads, rank + rot_dim]")
    if latent_out is not None:
        _require(write_rows and latent_out.shape == (tokens, rank) and latent_out.is_contiguous() and latent_out.dtype == q.dtype,
                 "the latents must be [tokens, rank]")
    _require(rotary_dim % 2 == 0 and 0 <= rotary_dim <= rot_dim, "rotary_dim must be even and at most rot_dim")
    if rotary_dim:
        _f32_vector(inv_freq, rotary_dim // 2, "the rotation's frequencies")
    _int_vector(positions, "positions")
    _int_vector(token_seq, "token_seq")
    if write_rows:
        _require(down.shape == (tokens, width) and down.dtype == q.dtype, "the down-projection must be [tokens, rank + rot_dim]")
        _require(rows.shape[1:] == (PAGE_TOKENS, width) and rows.is_contiguous() and rows.dtype == q.dtype, "cache rows must be [pages, 64, rank + rot_dim]")
        _f32_vector(latent_weight, rank, "the latent norm weight")
        _require(page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous(), "page rows must be int32 [sequences, stride]")
    library = build.load_library("latent_attention.cu")
    _check(library.tau_latent_prepare(
        _code(q), _pointer(down), ctypes.c_longlong(down.stride(0) if write_rows else 0), _pointer(latent_weight), ctypes.c_float(eps), _pointer(q),
        ctypes.c_longlong(q.stride(0)), _pointer(queries), _pointer(rows), _pointer(inv_freq), ctypes.c_int(rotary_dim), _pointer(positions),
        _pointer(token_seq), _pointer(page_rows), ctypes.c_int(page_rows.shape[1]), ctypes.c_int(PAGE_TOKENS), ctypes.c_int(tokens),
        ctypes.c_int(n_heads), ctypes.c_int(head_dim), ctypes.c_int(rot_dim), ctypes.c_int(rank), ctypes.c_int(1 if write_rows else 0),
        _pointer(latent_out), _stream()), "latent_prepare")


def latent_expand(q, down, expanded, queries, key_pages, value_pages, inv_freq, rotary_dim: int, positions, token_seq, pages_per_sequence: int,
                  n_heads: int, head_dim: int, rot_dim: int, rank: int, value_dim: int) -> None:
    """For runs that start at position 0: writes every head's query `[unrotated | rotated]` to `queries` [tokens, n_heads,
    head_dim + rot_dim], its key `[expanded unrotated part | rotated shared part]` and its value `[expanded | zeros]` to pages
    of their own ([sequences * pages_per_sequence, n_heads, 64, head_dim + rot_dim]; sequence `s` owns the pages from
    `s * pages_per_sequence`).  `expanded` [tokens, n_heads * (head_dim + value_dim)] holds all heads' unrotated keys, then all
    heads' values; `down` [tokens, rank + rot_dim] the shared key part behind the latent; `q` the projected queries."""
    _on_device(q, down, expanded, queries, key_pages, value_pages, inv_freq, positions, token_seq)
    tokens, width = q.shape[0], head_dim + rot_dim
    _require(q.shape[1] == n_heads * width and down.shape == (tokens, rank + rot_dim) and expanded.shape == (tokens, n_heads * (head_dim + value_dim))
             and expanded.is_contiguous(), "q, down and expanded must be [tokens, heads * (d + r)], [tokens, rank + r], [tokens, heads * (d + v)]")
    _require(queries.shape == (tokens, n_heads, width) and queries.is_contiguous(), "queries must be [tokens, n_heads, head_dim + rot_dim]")
    _require(key_pages.shape[1:] == (n_heads, PAGE_TOKENS, width) and key_pages.shape == value_pages.shape and key_pages.is_contiguous()
             and value_pages.is_contiguous() and key_pages.shape[0] % pages_per_sequence == 0, "pages must be [sequences * pages, n_heads, 64, width]")
    _require(q.dtype == down.dtype == expanded.dtype == queries.dtype == key_pages.dtype == value_pages.dtype, "one dtype throughout")
    _require(value_dim <= width and rotary_dim % 2 == 0 and rotary_dim <= rot_dim, "values may not be wider than keys")
    if rotary_dim:
        _f32_vector(inv_freq, rotary_dim // 2, "the rotation's frequencies")
    _int_vector(positions, "positions")
    _int_vector(token_seq, "token_seq")
    library = build.load_library("latent_attention.cu")
    _check(library.tau_latent_expand(
        _code(q), _pointer(q), ctypes.c_longlong(q.stride(0)), _pointer(down), ctypes.c_longlong(down.stride(0)), _pointer(expanded), _pointer(queries),
        _pointer(key_pages), _pointer(value_pages), _pointer(inv_freq), ctypes.c_int(rotary_dim), _pointer(positions), _pointer(token_seq),
        ctypes.c_int(pages_per_sequence), ctypes.c_int(PAGE_TOKENS), ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(head_dim),
        ctypes.c_int(rot_dim), ctypes.c_int(rank), ctypes.c_int(value_dim), _stream()), "latent_expand")


def head_gate(values, gate, out, n_heads: int, width: int, value_dim: int) -> None:
    """`out[token, head, :] = values[token, head, :value_dim] * sigmoid(gate[token, head, :])`: `values` [tokens, n_heads * width],
    `gate` [tokens, n_heads * value_dim] (rows any distance apart) or None, `out` [tokens, n_heads * value_dim]."""
    _on_device(values, gate, out)
    tokens = values.shape[0]
    _require(values.shape == (tokens, n_heads * width) and values.is_contiguous() and out.shape == (tokens, n_heads * value_dim) and out.is_contiguous()
             and out.dtype == values.dtype and value_dim <= width, "values must be [tokens, heads * width] and the output [tokens, heads * value_dim]")
    if gate is not None:
        _require(gate.shape == out.shape and gate.dtype == out.dtype and gate.stride(1) == 1, "the gate must match the output")
    library = build.load_library("latent_attention.cu")
    _check(library.tau_head_gate(_code(values), _pointer(values), _pointer(gate), ctypes.c_longlong(0 if gate is None else gate.stride(0)), _pointer(out),
                                 ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(width), ctypes.c_int(value_dim), _stream()), "latent_expand")


LATENT_MAX_RANK = 1024   # what the latent attention kernel keeps per lane (rows of up to 768 elements take the vector form)


_latent_scratch = {}
_latent_scratch_kept = []


def latent_attention(queries, rows, out, sinks, positions, token_seq, page_rows, n_heads: int, rank: int, rot_dim: int, scale: float,
                     window: int = 0, splits: int = 1) -> None:
    """Causal softmax attention of `queries` [tokens, n_heads, rank + rot_dim] over the cached rows [pages, 64, rank + rot_dim]
    of each token's sequence; a score is the dot product of a query with a row times `scale`; `out` [tokens, n_heads, rank]
    receives the weighted sums of the rows' first `rank` elements.  `sinks` (float32 [n_heads] or None): `exp(sink)` joins
    the softmax denominator.  Scores, weights and sums are 32-bit.  `splits` > 1 cuts every token's context into that many
    ranges, one block each, whose results a second kernel joins (for steps of few tokens over long contexts); rows that are
    not whole 16-byte vectors are served by a kernel that does not split."""
    _on_device(queries, rows, out, sinks, positions, token_seq, page_rows)
    tokens, width = queries.shape[0], rank + rot_dim
    _require(queries.shape == (tokens, n_heads, width) and queries.is_contiguous() and out.shape == (tokens, n_heads, rank) and out.is_contiguous()
             and out.dtype == queries.dtype == rows.dtype, "queries must be [tokens, n_heads, rank + rot_dim] and the output [tokens, n_heads, rank]")
    _require(rows.shape[1:] == (PAGE_TOKENS, width) and rows.is_contiguous(), "cache rows must be [pages, 64, rank + rot_dim]")
    _require(rank <= LATENT_MAX_RANK, f"the latent may have at most {LATENT_MAX_RANK} elements")
    _f32_vector(sinks, n_heads, "the sinks")
    _int_vector(positions, "positions")
    _int_vector(token_seq, "token_seq")
    _require(page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous(), "page rows must be int32 [sequences, stride]")
    _require(1 <= splits <= 64, "splits must lie between 1 and 64")
    library = build.load_library("latent_attention.cu")
    library.tau_latent_attention_scratch.restype = ctypes.c_longlong
    floats = library.tau_latent_attention_scratch(ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(rank), ctypes.c_int(splits))
    scratch = None
    if floats:
        key = (out.device, _stream_handle())
        scratch = _latent_scratch.get(key)
        if scratch is None or scratch.numel() < floats:
            if scratch is not None:
                _latent_scratch_kept.append(scratch)     # a captured graph may still name it
            scratch = _latent_scratch[key] = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=out.device)
    _check(library.tau_latent_attention(
        _code(queries), _pointer(queries), _pointer(rows), _pointer(out), _pointer(sinks), _pointer(positions), _pointer(token_seq),
        _pointer(page_rows), ctypes.c_int(page_rows.shape[1]), ctypes.c_int(PAGE_TOKENS), ctypes.c_int(tokens), ctypes.c_int(n_heads),
        ctypes.c_int(rank), ctypes.c_int(rot_dim), ctypes.c_float(scale), ctypes.c_int(window), ctypes.c_int(splits), _pointer(scratch),
        ctypes.c_longlong(0 if scratch is None else scratch.numel()), _stream()), "latent_attention", 2 if splits > 1 else 1)


# ---------------------------------------------------------------------------- differential attention
DIFF_MAX_VALUE_DIM = 512


def diff_prepare(projected, q_weight, k_weight, eps: float, inv_freq, rotary_dim: int, queries, rows, positions, token_seq, page_rows,
                 n_heads: int, n_kv_heads: int, dim: int, vdim: int, write_rows: bool = True) -> None:
    """`projected` [tokens, >= n_heads * 2 * dim + n_kv_heads * (2 * dim + vdim)] holds, per token, the two query maps of every head,
    the two key maps of every key/value head and the values.  Every map is divided by its root mean square over `dim` (eps inside
    the root), multiplied by `q_weight` or `k_weight` (float32 [dim]) and its first `rotary_dim` elements are turned pair by pair
    (2i, 2i + 1) by `position * inv_freq[i]`.  Queries go to `queries` [tokens, n_heads, 2, dim]; with `write_rows` keys and values
    go to the token's row of the cache pages `rows` [pages, 64, n_kv_heads * (2 * dim + vdim)] as [keys of all heads | values]."""
    _on_device(projected, q_weight, k_weight, inv_freq, queries, rows, positions, token_seq, page_rows)
    tokens = projected.shape[0]
    row_width = n_kv_heads * (2 * dim + vdim)
    _require(projected.shape[1] >= n_heads * 2 * dim + row_width and projected.stride(1) == 1, "the projection is too narrow")
    _require(queries.shape == (tokens, n_heads, 2, dim) and queries.is_contiguous() and queries.dtype == projected.dtype, "queries must be [tokens, n_heads, 2, dim]")
    _f32_vector(q_weight, dim, "the query norm weight")
    _f32_vector(k_weight, dim, "the key norm weight")
    _require(rotary_dim % 2 == 0 and 0 <= rotary_dim <= dim, "rotary_dim must be even and at most dim")
    if rotary_dim:
        _f32_vector(inv_freq, rotary_dim // 2, "the rotation's frequencies")
    _int_vector(positions, "positions")
    if write_rows:
        _int_vector(token_seq, "token_seq")
        _require(rows.shape[1:] == (PAGE_TOKENS, row_width) and rows.is_contiguous() and rows.dtype == projected.dtype, "cache rows must be [pages, 64, row width]")
        _require(page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous(), "page rows must be int32 [sequences, stride]")
    library = build.load_library("diff_attention.cu")
    _check(library.tau_diff_prepare(
        _code(projected), _pointer(projected), ctypes.c_longlong(projected.stride(0)), _pointer(q_weight), _pointer(k_weight), ctypes.c_float(eps),
        _pointer(inv_freq), ctypes.c_int(rotary_dim), _pointer(queries), _pointer(rows if write_rows else None), _pointer(positions), _pointer(token_seq),
        _pointer(page_rows), ctypes.c_int(page_rows.shape[1] if write_rows else 0), ctypes.c_int(PAGE_TOKENS), ctypes.c_int(tokens), ctypes.c_int(n_heads),
        ctypes.c_int(n_kv_heads), ctypes.c_int(dim), ctypes.c_int(vdim), ctypes.c_int(1 if write_rows else 0), _stream()), "diff_prepare")


def diff_attention(queries, rows, gate, out, step, page_rows, n_kv_heads: int, vdim: int, scale: float, window: int, lam: float, eps: float,
                   post_scale: float) -> None:
    """Two causal softmax maps per head over the cached rows of each token's sequence (within `window` positions if it is not 0):
    `o = a1 - lam * a2`, divided by its root mean square over the head's `vdim` values (eps inside the root), times `post_scale`,
    times `sigmoid(gate)` (`gate` [tokens, n_heads * vdim], rows any distance apart, or None); `out` [tokens, n_heads * vdim].
    Scores, weights, sums and the norm are 32-bit."""
    _on_device(queries, rows, gate, out, page_rows)
    tokens, n_heads, _, dim = queries.shape
    row_width = n_kv_heads * (2 * dim + vdim)
    _require(queries.is_contiguous() and out.shape == (tokens, n_heads * vdim) and out.is_contiguous() and out.dtype == queries.dtype == rows.dtype,
             "queries must be [tokens, n_heads, 2, dim] and the output [tokens, n_heads * vdim]")
    _require(rows.shape[1:] == (PAGE_TOKENS, row_width) and rows.is_contiguous(), "cache rows must be [pages, 64, row width]")
    _require(vdim <= DIFF_MAX_VALUE_DIM, f"values may have at most {DIFF_MAX_VALUE_DIM} elements per head")
    if gate is not None:
        _require(gate.shape == out.shape and gate.dtype == out.dtype and gate.stride(1) == 1, "the gate must have the output's shape and dtype")
    _require(page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous(), "page rows must be int32 [sequences, stride]")
    library = build.load_library("diff_attention.cu")
    _check(library.tau_diff_attention(
        _code(queries), _pointer(queries), _pointer(rows), _pointer(gate), ctypes.c_longlong(0 if gate is None else gate.stride(0)), _pointer(out),
        _pointer(step.positions), _pointer(step.token_seq), _pointer(page_rows), ctypes.c_int(page_rows.shape[1]), ctypes.c_int(PAGE_TOKENS),
        ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(dim), ctypes.c_int(vdim), ctypes.c_float(scale),
        ctypes.c_int(window), ctypes.c_float(lam), ctypes.c_float(eps), ctypes.c_float(post_scale), _stream()), "diff_attention")


def diff_prepare_wide(projected, q_weight, k_weight, eps: float, inv_freq, rotary_dim: int, queries, key_pages, value_pages, positions, token_seq,
                      page_rows, n_heads: int, n_kv_heads: int, dim: int, vdim: int, write_cache: bool = True) -> None:
    """As `diff_prepare`, for the cache of ordinary heads: every map becomes a head of `wide` = `queries.shape[2]` >= max(dim, vdim)
    elements, zeros behind what it holds.  `queries` [tokens, 2 * n_heads, wide] holds query (head, map) in slot
    `(group * 2 + map) * (n_heads / n_kv_heads) + head % (n_heads / n_kv_heads)`; `key_pages` and `value_pages`
    [pages, 2 * n_kv_heads, 64, wide] hold key (group, map) under head `group * 2 + map` and the group's values under both, so
    that grouped-query attention over 2 * n_heads heads and 2 * n_kv_heads key/value heads computes both maps of every head."""
    _on_device(projected, q_weight, k_weight, inv_freq, queries, key_pages, value_pages, positions, token_seq, page_rows)
    tokens, wide = projected.shape[0], queries.shape[2]
    _require(projected.shape[1] >= n_heads * 2 * dim + n_kv_heads * (2 * dim + vdim) and projected.stride(1) == 1, "the projection is too narrow")
    _require(queries.shape == (tokens, 2 * n_heads, wide) and queries.is_contiguous() and queries.dtype == projected.dtype and wide >= max(dim, vdim)
             and wide % 2 == 0, "queries must be [tokens, 2 * n_heads, wide]")
    _f32_vector(q_weight, dim, "the query norm weight")
    _f32_vector(k_weight, dim, "the key norm weight")
    _require(rotary_dim % 2 == 0 and 0 <= rotary_dim <= dim, "rotary_dim must be even and at most dim")
    if rotary_dim:
        _f32_vector(inv_freq, rotary_dim // 2, "the rotation's frequencies")
    _int_vector(positions, "positions")
    if write_cache:
        _int_vector(token_seq, "token_seq")
        for pages in (key_pages, value_pages):
            _require(pages.shape[1:] == (2 * n_kv_heads, PAGE_TOKENS, wide) and pages.is_contiguous() and pages.dtype == projected.dtype,
                     "cache pages must be [pages, 2 * n_kv_heads, 64, wide]")
        _require(page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous(), "page rows must be int32 [sequences, stride]")
    library = build.load_library("diff_attention.cu")
    _check(library.tau_diff_prepare_wide(
        _code(projected), _pointer(projected), ctypes.c_longlong(projected.stride(0)), _pointer(q_weight), _pointer(k_weight), ctypes.c_float(eps),
        _pointer(inv_freq), ctypes.c_int(rotary_dim), _pointer(queries), _pointer(key_pages if write_cache else None),
        _pointer(value_pages if write_cache else None), _pointer(positions), _pointer(token_seq), _pointer(page_rows),
        ctypes.c_int(page_rows.shape[1] if write_cache else 0), ctypes.c_int(PAGE_TOKENS), ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads),
        ctypes.c_int(dim), ctypes.c_int(vdim), ctypes.c_int(wide), ctypes.c_int(1 if write_cache else 0), _stream()), "diff_prepare")


def diff_combine(attended, gate, out, n_heads: int, n_kv_heads: int, vdim: int, lam: float, eps: float, post_scale: float) -> None:
    """`attended` [tokens, 2 * n_heads, wide] in the slots of `diff_prepare_wide`: per head `o = map 1 - lam * map 2` over the first
    `vdim` elements, divided by its root mean square (eps inside the root), times `post_scale`, times `sigmoid(gate)` (or no gate);
    `out` [tokens, n_heads * vdim].  32-bit throughout, one rounding."""
    _on_device(attended, gate, out)
    tokens, _, wide = attended.shape
    _require(attended.shape[1] == 2 * n_heads and attended.is_contiguous() and out.shape == (tokens, n_heads * vdim) and out.is_contiguous()
             and out.dtype == attended.dtype, "attended must be [tokens, 2 * n_heads, wide] and the output [tokens, n_heads * vdim]")
    _require(vdim <= DIFF_MAX_VALUE_DIM and vdim <= wide, f"values may have at most {DIFF_MAX_VALUE_DIM} elements per head")
    if gate is not None:
        _require(gate.shape == out.shape and gate.dtype == out.dtype and gate.stride(1) == 1, "the gate must have the output's shape and dtype")
    library = build.load_library("diff_attention.cu")
    _check(library.tau_diff_combine(_code(out), _pointer(attended), _pointer(gate), ctypes.c_longlong(0 if gate is None else gate.stride(0)), _pointer(out),
                                    ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(vdim), ctypes.c_int(wide),
                                    ctypes.c_float(lam), ctypes.c_float(eps), ctypes.c_float(post_scale), _stream()), "diff_combine")


# ---------------------------------------------------------------------------- sublayer arrangement on a 32-bit stream
def causal_taps(stream, weight, state, step, read_out, plain_out=None, update: bool = True) -> None:
    """`read_out[t] = stream[t] + sum_j weight[j] * stream[t - taps + 1 + j]` (`weight` float32 [taps, width]: tap by tap, so that a
    tap's channels lie side by side) over each sequence's run of the step, the rows before
    the run's first token taken from `state[slot]` ([slots, taps - 1, width] float32: the sequence's last inputs, zeros at its start);
    `plain_out` (optional) receives `stream` itself in the output's dtype.  With `update` the state then becomes the last `taps - 1`
    inputs of each sequence (a second launch, or the same one where every sequence brings one token)."""
    _on_device(stream, weight, state, read_out, plain_out)
    tokens, width = stream.shape
    taps = 0 if weight is None else weight.shape[0]      # without a weight the outputs are the stream itself, rounded
    _require(stream.dtype == torch.float32 and stream.is_contiguous(), "the stream must be contiguous float32")
    if weight is not None:
        _require(weight.dtype == torch.float32 and weight.shape == (taps, width) and weight.is_contiguous() and taps >= 1, "the taps must be float32 [taps, width]")
    if taps > 1:
        _require(state is not None and state.dtype == torch.float32 and state.shape[1:] == (taps - 1, width) and state.is_contiguous(),
                 "the state must be float32 [slots, taps - 1, width]")
    update = update and taps > 1
    _require(read_out.shape == stream.shape and read_out.is_contiguous(), "the output must match the stream")
    if plain_out is not None:
        _require(plain_out.shape == stream.shape and plain_out.is_contiguous() and plain_out.dtype == read_out.dtype, "the plain output must match the other")
    single = bool(getattr(step, "all_single", False)) and tokens == step.n_seqs
    library = build.load_library("sublayer.cu")
    _check(library.tau_causal_taps(_code(read_out), _pointer(stream), _pointer(weight), _pointer(state), _pointer(step.token_seq), _pointer(step.cu_seqlens),
                                   _pointer(step.seq_slot), _pointer(read_out), _pointer(plain_out), ctypes.c_int(tokens), ctypes.c_int(step.n_seqs),
                                   ctypes.c_int(width), ctypes.c_int(taps), ctypes.c_int(1 if update else 0), ctypes.c_int(1 if single else 0), _stream()),
           "causal_taps", 2 if update and not single else 1)


def gated_add_norm(source, target, branch, gate, weight, bias, eps: float, centred: bool, copy_out=None) -> None:
    """`target = source + norm(branch * sigmoid(gate)) * weight + bias` row by row on a 32-bit stream (`target` may be `source`):
    the norm subtracts the mean and divides by the root of the variance plus eps (`centred`, a layer norm) or divides by the root of
    the mean square plus eps.  `gate` (rows any distance apart) and `bias` may be None.  `copy_out` receives the new rows rounded."""
    _on_device(source, target, branch, gate, weight, bias, copy_out)
    rows, width = source.shape
    _require(source.dtype == target.dtype == torch.float32 and source.is_contiguous() and target.is_contiguous() and target.shape == source.shape,
             "source and target must be contiguous float32 of one shape")
    _require(branch.shape == source.shape and branch.is_contiguous(), "the branch must match the stream")
    if gate is not None:
        _require(gate.shape == source.shape and gate.stride(1) == 1, "the gate must match the stream")
    _f32_vector(weight, width, "the norm weight")
    _f32_vector(bias, width, "the norm bias")
    if copy_out is not None:
        _require(copy_out.shape == source.shape and copy_out.is_contiguous(), "the copy must match the stream")
    library = build.load_library("sublayer.cu")
    _check(library.tau_gated_add_norm(_code(copy_out) if copy_out is not None else 0, _pointer(source), _pointer(target), _pointer(branch), ctypes.c_int(_code(branch)),
                                      _pointer(gate), ctypes.c_int(_code(gate) if gate is not None else 0), ctypes.c_longlong(0 if gate is None else gate.stride(0)),
                                      _pointer(weight), _pointer(bias), _pointer(copy_out), ctypes.c_int(rows), ctypes.c_int(width), ctypes.c_float(eps),
                                      ctypes.c_int(1 if centred else 0), _stream()), "gated_add_norm")


def side_gate(z, table, token_ids, offset: int, out) -> None:
    """`out[t, c] = gelu_tanh(z[t, c]) * table[token_ids[t], offset + c]`, the tanh form of GELU in 32-bit."""
    _on_device(z, table, token_ids, out)
    rows, dim = z.shape
    _require(z.is_contiguous() and out.is_contiguous() and out.shape == z.shape and out.dtype == z.dtype == table.dtype and table.is_contiguous(),
             "z, the table and the output must be contiguous and of one dtype")
    _require(0 <= offset and offset + dim <= table.shape[1], "the table has no such columns")
    _int_vector(token_ids, "token ids")
    library = build.load_library("sublayer.cu")
    _check(library.tau_side_gate(_code(z), _pointer(z), _pointer(table), _pointer(token_ids), _pointer(out), ctypes.c_int(rows), ctypes.c_int(dim),
                                 ctypes.c_int(table.shape[1]), ctypes.c_int(offset), ctypes.c_int(table.shape[0]), _stream()), "side_gate")


def unit_add_mix(source, y, weight, eps: float, result, results=None, mix=None, out=None, copy_out=None) -> None:
    """`result = source + y / sqrt(mean(y^2) + eps) * weight` row by row on a 32-bit stream (`result = source` if `y` is None).  With `mix` (float32 [count]) and
    `results` ([count - 1 or more, rows, width] float32: the earlier results, `result` being the newest) `out = sum_j mix[j] * results[j]`
    with `results[count - 1]` standing for `result`.  `copy_out` receives `out` (or `result`, without `mix`) rounded."""
    _on_device(source, y, weight, result, results, mix, out, copy_out)
    rows, width = source.shape
    _require(source.dtype == result.dtype == torch.float32 and source.is_contiguous() and result.is_contiguous() and result.shape == source.shape,
             "source and result must be contiguous float32 of one shape")
    if y is not None:
        _require(y.shape == source.shape and y.is_contiguous() and weight is not None, "y must match the stream and have a weight")
    _f32_vector(weight, width, "the norm weight")
    count = 0
    if mix is not None:
        count = mix.numel()
        _require(mix.dtype == torch.float32 and mix.is_contiguous() and count >= 1, "the mix must be a float32 vector")
        _require(out is not None and out.dtype == torch.float32 and out.shape == source.shape and out.is_contiguous(), "the mixed output must match the stream")
        if count > 1:
            _require(results is not None and results.dtype == torch.float32 and results.shape[0] >= count - 1 and results.shape[1:] == source.shape
                     and results.is_contiguous(), "results must be float32 [count - 1 or more, rows, width]")
    if copy_out is not None:
        _require(copy_out.shape == source.shape and copy_out.is_contiguous(), "the copy must match the stream")
    library = build.load_library("sublayer.cu")
    _check(library.tau_unit_add_mix(_code(copy_out) if copy_out is not None else 0, _pointer(source), _pointer(y), ctypes.c_int(_code(y) if y is not None else 0), _pointer(weight),
                                    _pointer(result), _pointer(results), ctypes.c_longlong(rows * width), _pointer(mix), ctypes.c_int(count), _pointer(out),
                                    _pointer(copy_out), ctypes.c_int(rows), ctypes.c_int(width), ctypes.c_float(eps), _stream()), "unit_add_mix")


def norm_rows(values, rows, weight, bias, eps: float, centred: bool, out) -> None:
    """`out[i] = norm(values[rows[i]]) * weight + bias` (`rows` None: every row): a layer norm (`centred`) or an RMS norm, in 32-bit."""
    _on_device(values, rows, weight, bias, out)
    width = values.shape[-1]
    _require(values.is_contiguous() and out.is_contiguous() and out.shape[-1] == width, "input and output must be contiguous and as wide")
    _f32_vector(weight, width, "the norm weight")
    _f32_vector(bias, width, "the norm bias")
    if rows is not None:
        _int_vector(rows, "row numbers")
    count = out.numel() // width
    _require(count == (rows.shape[0] if rows is not None else values.numel() // width), "output row count does not match")
    library = build.load_library("sublayer.cu")
    _check(library.tau_norm_rows(_code(out), _pointer(values), ctypes.c_int(_code(values)), _pointer(rows), _pointer(weight), _pointer(bias), _pointer(out),
                                 ctypes.c_int(count), ctypes.c_int(width), ctypes.c_float(eps), ctypes.c_int(1 if centred else 0), _stream()), "norm_rows")


def relu_squared(z, out) -> None:
    """`out = max(z, 0)^2`."""
    _on_device(z, out)
    _require(z.is_contiguous() and out.is_contiguous() and z.shape == out.shape and z.dtype == out.dtype, "input and output must match")
    library = build.load_library("sublayer.cu")
    _check(library.tau_relu_squared(_code(z), _pointer(z), _pointer(out), ctypes.c_longlong(z.numel()), _stream()), "relu_squared")


# ---------------------------------------------------------------------------- linear recurrences
RECURRENCE_MAX_KEY_DIM = 512


def linear_recurrence(q, k, v, gates, decays, state, cu_seqlens, seq_slot, out, n_heads: int, key_dim: int, value_dim: int,
                      exponential: bool, gate_cap: float = 0.0, query_scale: float = 1.0, silu: bool = False) -> None:
    """Advances the matrix state of every (sequence, head) over the sequence's new tokens and writes each token's read-out.

    `q`, `k` [tokens, n_heads * key_dim] and `v` [tokens, n_heads * value_dim] may be column ranges of one wider tensor (same
    row stride).  `state` [slots, floats per slot] is 32-bit and updated in place: per head `value_dim` columns of `key_dim`
    numbers, and with `exponential` one more column (the normaliser) and the running maximum.  `gates` [tokens, 2 * n_heads]
    float32 are the pre-activations of the input gates, then of the forget gates (overwritten with the log gates);
    `decays` [n_heads] float32 otherwise.
    `out` [tokens, n_heads * value_dim] float32."""
    _on_device(q, k, v, gates, decays, state, cu_seqlens, seq_slot, out)
    tokens = q.shape[0]
    _require(q.shape == (tokens, n_heads * key_dim) == k.shape and v.shape == (tokens, n_heads * value_dim), "q, k must be [tokens, heads * key_dim], v [tokens, heads * value_dim]")
    _require(q.dtype == k.dtype == v.dtype and q.stride(0) == k.stride(0) == v.stride(0), "q, k and v must share dtype and row stride")
    _require(1 <= key_dim <= RECURRENCE_MAX_KEY_DIM, f"key_dim must lie between 1 and {RECURRENCE_MAX_KEY_DIM}")
    per_head = (value_dim + 1) * key_dim + 1 if exponential else value_dim * key_dim
    _require(state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous() and state.shape[1] == n_heads * per_head,
             f"the state must be float32 [slots, {n_heads * per_head}]")
    _require(out.shape == (tokens, n_heads * value_dim) and out.dtype == torch.float32 and out.is_contiguous(), "the output must be float32 [tokens, heads * value_dim]")
    if exponential:
        _require(gates is not None and gates.shape == (tokens, 2 * n_heads) and gates.dtype == torch.float32 and gates.is_contiguous(),
                 "gates must be float32 [tokens, 2 * heads]")
    else:
        _f32_vector(decays, n_heads, "the decays")
        _require(decays is not None, "decays are needed")
    _int_vector(cu_seqlens, "cu_seqlens")
    _int_vector(seq_slot, "seq_slot")
    n_seqs = seq_slot.numel()
    _require(cu_seqlens.numel() == n_seqs + 1, "one run per sequence")
    library = build.load_library("recurrence.cu", (f"TAU_KEY_DIM={key_dim}",))
    _check(library.tau_linear_recurrence(
        _code(q), _pointer(q), _pointer(k), _pointer(v), ctypes.c_longlong(q.stride(0)), _pointer(gates), _pointer(decays), _pointer(state),
        ctypes.c_longlong(state.stride(0)), _pointer(cu_seqlens), _pointer(seq_slot), _pointer(out), ctypes.c_int(tokens), ctypes.c_int(n_seqs), ctypes.c_int(n_heads),
        ctypes.c_int(value_dim), ctypes.c_int(1 if exponential else 0), ctypes.c_float(gate_cap), ctypes.c_float(query_scale),
        ctypes.c_int(1 if silu else 0), _stream()), "linear_recurrence", 2 if exponential else 1)


# ---------------------------------------------------------------------------- short convolutions, delta rule, selective scan
def short_conv(x, weight, bias, state, step, out, silu: bool = True, update: bool = True) -> None:
    """`out[t, c] = act(bias[c] + sum_j weight[j, c] * x[t - (taps - 1) + j, c])` over each sequence's run of the step (`weight`
    float32 [taps, channels], tap by tap, the last tap weighing the token itself; `bias` float32 [channels] or None; `act` SiLU or
    none); rows before the run's first token come from `state[slot]` ([slots, taps - 1, channels] float32: the sequence's last
    inputs, zeros at its start).  `x` and `out` may be column ranges of wider tensors; `out` is float32 or of `x`'s dtype.  With
    `update` the state then becomes the last `taps - 1` inputs of each sequence (a second launch, or the same one where every
    sequence brings one token)."""
    _on_device(x, weight, bias, state, out)
    tokens, channels = x.shape
    taps = weight.shape[0]
    _require(x.stride(1) == 1 and out.stride(1) == 1 and out.shape == x.shape and out.dtype in (torch.float32, x.dtype), "the output must match the input's shape")
    _require(weight.dtype == torch.float32 and weight.shape == (taps, channels) and weight.is_contiguous() and taps >= 1, "the taps must be float32 [taps, channels]")
    _f32_vector(bias, channels, "the bias")
    if taps > 1:
        _require(state is not None and state.dtype == torch.float32 and state.shape[1:] == (taps - 1, channels) and state.is_contiguous(),
                 "the state must be float32 [slots, taps - 1, channels]")
    update = update and taps > 1
    single = bool(getattr(step, "all_single", False)) and tokens == step.n_seqs
    library = build.load_library("short_conv.cu")
    _check(library.tau_short_conv(_code(x), _code(out), _pointer(x), ctypes.c_longlong(x.stride(0)), _pointer(weight), _pointer(bias), _pointer(state),
                                  _pointer(step.token_seq), _pointer(step.cu_seqlens), _pointer(step.seq_slot), _pointer(out), ctypes.c_longlong(out.stride(0)),
                                  ctypes.c_int(tokens), ctypes.c_int(step.n_seqs), ctypes.c_int(channels), ctypes.c_int(taps), ctypes.c_int(1 if silu else 0),
                                  ctypes.c_int(1 if update else 0), ctypes.c_int(1 if single else 0), _stream()),
           "short_conv", 2 if update and not single else 1)


DELTA_MAX_KEY_DIM = 512


def delta_prepare(rows, q_offset: int, k_offset: int, pre, a_log, dt_bias, gates, kq, n_heads: int, n_key_heads: int, key_dim: int, channel=None) -> None:
    """In place on `rows` (float32 [tokens, width]): the queries (`n_key_heads * key_dim` columns from `q_offset`) and keys (from
    `k_offset`) become unit vectors per head, `x / sqrt(sum(x^2) + 1e-6)`, the queries also times `key_dim ** -0.5`.
    `kq` [tokens, n_key_heads] receives `k . q` of the results.  `pre` float32 [tokens, 2 * n_heads] holds per value head the
    pre-activation of beta, then of the decay's step; `gates` [tokens, n_heads, 2] receives
    `(exp(-exp(a_log) * softplus(step + dt_bias)), sigmoid(beta))`.  With `channel` (float32 [tokens, n_heads * key_dim]: the
    pre-activations of a decay per head and key channel) `pre` holds beta's alone ([tokens, n_heads]), `dt_bias` is as wide as
    `channel`, and `channel` is replaced by `exp(-exp(a_log[head]) * softplus(channel + dt_bias))`."""
    _on_device(rows, pre, a_log, dt_bias, gates, kq, channel)
    tokens = rows.shape[0]
    _require(rows.dtype == torch.float32 and rows.stride(1) == 1 and max(q_offset, k_offset) + n_key_heads * key_dim <= rows.shape[1], "rows must be float32 and hold q and k")
    _require(pre.dtype == torch.float32 and pre.dim() == 2 and pre.shape[0] == tokens and pre.shape[1] >= (1 if channel is not None else 2) * n_heads
             and pre.stride(1) == 1, "the gates' pre-activations must be float32 [tokens, 2 * heads] (beta's alone beside a decay per channel)")
    _f32_vector(a_log, n_heads, "A_log")
    _f32_vector(dt_bias, n_heads * (key_dim if channel is not None else 1), "dt_bias")
    if channel is not None:
        _require(channel.dtype == torch.float32 and channel.shape == (tokens, n_heads * key_dim) and channel.is_contiguous(), "the decays must be float32 [tokens, heads * key_dim]")
    _require(gates.dtype == torch.float32 and gates.shape == (tokens, n_heads, 2) and gates.is_contiguous(), "gates must be float32 [tokens, heads, 2]")
    _require(kq.dtype == torch.float32 and kq.shape == (tokens, n_key_heads) and kq.is_contiguous(), "kq must be float32 [tokens, key heads]")
    _require(1 <= key_dim <= DELTA_MAX_KEY_DIM and n_heads % n_key_heads == 0, f"key_dim must lie between 1 and {DELTA_MAX_KEY_DIM}, and the key heads divide the heads")
    library = build.load_library("delta_rule.cu", (f"TAU_KEY_DIM={key_dim}",))
    _check(library.tau_delta_prepare(_pointer(rows), ctypes.c_longlong(rows.stride(0)), ctypes.c_int(q_offset), ctypes.c_int(k_offset), _pointer(pre),
                                     ctypes.c_int(pre.stride(0)), _pointer(a_log), _pointer(dt_bias), _pointer(gates), _pointer(kq), _pointer(channel), ctypes.c_int(tokens), ctypes.c_int(n_heads),
                                     ctypes.c_int(n_key_heads), ctypes.c_float(key_dim ** -0.5), _stream()), "delta_prepare")


def delta_rule(rows, q_offset: int, k_offset: int, v_offset: int, gates, kq, state, cu_seqlens, seq_slot, out, n_heads: int, n_key_heads: int,
               key_dim: int, value_dim: int, channel=None) -> None:
    """Advances the gated delta rule of every (sequence, head) over the sequence's new tokens: `S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q`.  `rows` as `delta_prepare` left them, with the values (`n_heads * value_dim` columns) from
    `v_offset`; `gates` [tokens, n_heads, 2] = (g, beta); `kq` [tokens, n_key_heads]; `state` float32 [slots, n_heads * value_dim *
    key_dim], updated in place; `out` float32 [tokens, n_heads * value_dim].  `channel` (float32 [tokens, n_heads * key_dim], as
    `delta_prepare` left it): g is that vector over the state's rows instead of the head's one number."""
    _on_device(rows, gates, kq, state, cu_seqlens, seq_slot, out, channel)
    if channel is not None:
        _require(channel.dtype == torch.float32 and channel.shape == (rows.shape[0], n_heads * key_dim) and channel.is_contiguous(), "the decays must be float32 [tokens, heads * key_dim]")
    tokens = rows.shape[0]
    _require(rows.dtype == torch.float32 and rows.stride(1) == 1 and v_offset + n_heads * value_dim <= rows.shape[1], "rows must be float32 and hold q, k and v")
    _require(gates.dtype == torch.float32 and gates.shape == (tokens, n_heads, 2) and gates.is_contiguous(), "gates must be float32 [tokens, heads, 2]")
    _require(kq.dtype == torch.float32 and kq.shape == (tokens, n_key_heads) and kq.is_contiguous(), "kq must be float32 [tokens, key heads]")
    _require(state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous() and state.shape[1] == n_heads * value_dim * key_dim,
             f"the state must be float32 [slots, {n_heads * value_dim * key_dim}]")
    _require(out.shape == (tokens, n_heads * value_dim) and out.dtype == torch.float32 and out.is_contiguous(), "the output must be float32 [tokens, heads * value_dim]")
    _require(1 <= key_dim <= DELTA_MAX_KEY_DIM and n_heads % n_key_heads == 0, f"key_dim must lie between 1 and {DELTA_MAX_KEY_DIM}, and the key heads divide the heads")
    _int_vector(cu_seqlens, "cu_seqlens")
    _int_vector(seq_slot, "seq_slot")
    n_seqs = seq_slot.numel()
    _require(cu_seqlens.numel() == n_seqs + 1, "one run per sequence")
    library = build.load_library("delta_rule.cu", (f"TAU_KEY_DIM={key_dim}",))
    _check(library.tau_delta_rule(_pointer(rows), ctypes.c_longlong(rows.stride(0)), ctypes.c_int(q_offset), ctypes.c_int(k_offset), ctypes.c_int(v_offset),
                                  _pointer(gates), _pointer(kq), _pointer(channel), _pointer(state), ctypes.c_longlong(state.stride(0)), _pointer(cu_seqlens), _pointer(seq_slot),
                                  _pointer(out), ctypes.c_int(n_seqs), ctypes.c_int(n_heads), ctypes.c_int(n_key_heads), ctypes.c_int(value_dim), _stream()),
           "delta_rule")


SCAN_MAX_STATES = 256


def selective_scan(x, z, pre, bc, a_log, skip, state, cu_seqlens, seq_slot, out) -> None:
    """Per channel `c` and state `n`, over each sequence's new tokens: `step = softplus(pre[t, c])`;
    `S[c, n] <- exp(step * A[c, n]) * S[c, n] + step * x[t, c] * B[t, n]` with `A = -exp(a_log)`; `y = sum_n S[c, n] * C[t, n] +
    skip[c] * x[t, c]`; `out[t, c] = y * silu(z[t, c])`.  `x`, `z` [tokens, channels] (column ranges of wider tensors allowed),
    `pre` float32 [tokens, channels], `bc` float32 [tokens, 2 * states] (B, then C), `a_log` float32 [channels, states],
    `state` float32 [slots, channels * states], updated in place; `out` [tokens, channels] of `x`'s dtype."""
    _on_device(x, z, pre, bc, a_log, skip, state, cu_seqlens, seq_slot, out)
    tokens, channels = x.shape
    states = a_log.shape[1]
    _require(x.stride(1) == 1 and z.stride(1) == 1 and z.shape == x.shape and z.dtype == x.dtype == out.dtype and out.shape == x.shape and out.is_contiguous(),
             "x, z and the output must be [tokens, channels] of one dtype")
    _require(pre.dtype == torch.float32 and pre.shape == x.shape and pre.is_contiguous(), "the steps' pre-activations must be float32 [tokens, channels]")
    _require(bc.dtype == torch.float32 and bc.shape == (tokens, 2 * states) and bc.is_contiguous(), "B and C must be float32 [tokens, 2 * states]")
    _require(a_log.dtype == torch.float32 and a_log.shape == (channels, states) and a_log.is_contiguous() and 1 <= states <= SCAN_MAX_STATES,
             f"A_log must be float32 [channels, states] with at most {SCAN_MAX_STATES} states")
    _f32_vector(skip, channels, "the skip weight")
    _require(state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous() and state.shape[1] == channels * states,
             f"the state must be float32 [slots, {channels * states}]")
    _int_vector(cu_seqlens, "cu_seqlens")
    _int_vector(seq_slot, "seq_slot")
    n_seqs = seq_slot.numel()
    _require(cu_seqlens.numel() == n_seqs + 1, "one run per sequence")
    library = build.load_library("selective_scan.cu", (f"TAU_SCAN_STATES={states}",))
    _check(library.tau_selective_scan(_code(x), _pointer(x), ctypes.c_longlong(x.stride(0)), _pointer(z), ctypes.c_longlong(z.stride(0)), _pointer(pre),
                                      _pointer(bc), _pointer(a_log), _pointer(skip), _pointer(state), _pointer(cu_seqlens), _pointer(seq_slot), _pointer(out),
                                      ctypes.c_int(n_seqs), ctypes.c_int(tokens), ctypes.c_int(channels), _stream()), "selective_scan")


# ---------------------------------------------------------------------------- attention over cached rows with a mask and a sink
MASKED_MAX_VALUE_DIM = 512
MASKED_STAGED_WARPS = 4      # query heads of a key/value head that one block of the staged kernel serves


def masked_prepare(projected, q_weight, k_weight, eps: float, frequency, rotary_dim: int, magnitude: float, queries, rows, positions, token_seq,
                   page_rows, n_heads: int, n_kv_heads: int, dim: int, vdim: int, write_rows: bool = True, value_pages=None,
                   temperature=None) -> None:
    """`projected` [tokens, >= n_heads * dim + n_kv_heads * (dim + vdim)] holds queries, keys and values side by side.  With weights
    (float32 [n_heads * dim] and [n_kv_heads * dim]) the queries, and the keys, are divided by the root mean square over their
    whole projection (eps inside the root) and multiplied by the weight.  In every head element `i` of the first `rotary_dim` is
    turned together with element `i + rotary_dim / 2` by `position * frequency[i]`, sine and cosine times `magnitude`.  Queries go
    to `queries` [tokens, n_heads, dim]; with `write_rows` keys and values go to the token's row of the cache pages `rows`
    [pages, 64, n_kv_heads * (dim + vdim)] as [keys of all heads | values], or, with `value_pages`, to pages of ordinary heads:
    keys to `rows` [pages, n_kv_heads, 64, dim], values to `value_pages` [pages, n_kv_heads, 64, vdim].  Without `write_rows` the
    projection need hold the queries alone.  `temperature` = (coef, every): the query at position p is multiplied by
    `1 + coef * ln(floor((p + 1) / every) + 1)`."""
    _on_device(projected, q_weight, k_weight, frequency, queries, rows, positions, token_seq, page_rows, value_pages)
    tokens = projected.shape[0]
    row_width = n_kv_heads * (dim + vdim)
    _require(projected.shape[1] >= n_heads * dim + (row_width if write_rows else 0) and projected.stride(1) == 1, "the projection is too narrow")
    coef, every = (0.0, 0) if temperature is None else (float(temperature[0]), int(temperature[1]))
    _require(every >= 0, "the temperature's period must be positive")
    _require(queries.shape == (tokens, n_heads, dim) and queries.is_contiguous() and queries.dtype == projected.dtype, "queries must be [tokens, n_heads, dim]")
    _f32_vector(q_weight, n_heads * dim, "the query norm weight")
    _f32_vector(k_weight, n_kv_heads * dim, "the key norm weight")
    _require(rotary_dim % 2 == 0 and 0 <= rotary_dim <= dim, "rotary_dim must be even and at most dim")
    if rotary_dim:
        _f32_vector(frequency, rotary_dim // 2, "the rotation's frequencies")
    _int_vector(positions, "positions")
    if write_rows:
        _int_vector(token_seq, "token_seq")
        _require_masked_pages(rows, value_pages, projected.dtype, n_kv_heads, dim, vdim)
        _require(page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous(), "page rows must be int32 [sequences, stride]")
    library = build.load_library("masked_attention.cu")
    _check(library.tau_masked_prepare(
        _code(projected), _pointer(projected), ctypes.c_longlong(projected.stride(0)), _pointer(q_weight), _pointer(k_weight), ctypes.c_float(eps),
        _pointer(frequency if rotary_dim else None), ctypes.c_int(rotary_dim), ctypes.c_float(magnitude), _pointer(queries), _pointer(rows if write_rows else None),
        _pointer(value_pages if write_rows else None), _pointer(positions), _pointer(token_seq), _pointer(page_rows), ctypes.c_int(page_rows.shape[1] if write_rows else 0), ctypes.c_int(PAGE_TOKENS),
        ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(dim), ctypes.c_int(vdim), ctypes.c_int(1 if write_rows else 0),
        ctypes.c_float(coef), ctypes.c_int(every), _stream()), "masked_prepare")


def _require_masked_pages(rows, value_pages, dtype, n_kv_heads: int, dim: int, vdim: int) -> None:
    if value_pages is None:
        _require(rows.shape[1:] == (PAGE_TOKENS, n_kv_heads * (dim + vdim)) and rows.is_contiguous() and rows.dtype == dtype, "cache rows must be [pages, 64, row width]")
    else:
        _require(rows.shape[1:] == (n_kv_heads, PAGE_TOKENS, dim) and value_pages.shape == (rows.shape[0], n_kv_heads, PAGE_TOKENS, vdim) and rows.is_contiguous()
                 and value_pages.is_contiguous() and rows.dtype == value_pages.dtype == dtype, "pages of heads must be [pages, kv heads, 64, dim] and [.., vdim]")


def masked_attention(queries, rows, out, step, page_rows, n_kv_heads: int, vdim: int, scale: float, window: int = 0, chunk: int = 0, sink: bool = False,
                     out_scale: float = 1.0, value_pages=None, staged: bool = False, distance=None, sigmoid_weights: bool = False, head_offset=None,
                     gate=None, gate_per_head: bool = False, splits: int = 1) -> None:
    """Causal softmax attention of every token over the cached rows of its sequence: within `window` positions (if not 0), or
    within the token's own chunk of `chunk` positions counted from position 0 (if not 0); with `sink` the softmax's denominator has
    one added.  `out` [tokens, n_heads * vdim] (rows any distance apart) receives the result times `out_scale`.  Scores, weights
    and sums are 32-bit.  The cache is `rows`, or `rows` and `value_pages` in the layout of ordinary heads (see `masked_prepare`).
    `staged` (meant for steps of single tokens) asks for the kernel that stages tiles of the cache in shared memory and shares them
    among the heads of a key/value head; sizes that it does not serve take the other kernel.  `distance` (float32 [n_heads, 2] =
    (r1, r2)): `r1 * ln(1 + r2 * (i - j))` is taken off the score of key j for the query at i.  `sigmoid_weights`: instead of a
    softmax every visible key weighs `sigmoid(score + head_offset[head])` (float32 [n_heads] or None), not normalised.  `gate`
    ([tokens, n_heads] with `gate_per_head`, else [tokens, n_heads * vdim]; the queries' dtype; rows any distance apart): the result
    is multiplied by its sigmoid.  `splits` > 1 (with `staged`): every token's context is cut into that many ranges that as many
    blocks walk, and a second launch joins them."""
    _on_device(queries, rows, out, page_rows, value_pages, distance, head_offset, gate)
    tokens, n_heads, dim = queries.shape
    if distance is not None:
        _require(distance.dtype == torch.float32 and distance.shape == (n_heads, 2) and distance.is_contiguous(), "the distance numbers must be float32 [heads, 2]")
    _f32_vector(head_offset, n_heads, "the heads' offsets")
    _require(not (sigmoid_weights and sink), "sigmoid weights have no denominator for a sink to join")
    if gate is not None:
        _require(gate.dtype == queries.dtype and gate.shape == (tokens, n_heads if gate_per_head else n_heads * vdim) and gate.stride(1) == 1,
                 "the gate must be [tokens, heads] or [tokens, heads * vdim] in the queries' dtype")
    _require(queries.is_contiguous() and out.shape == (tokens, n_heads * vdim) and out.stride(1) == 1 and out.dtype == queries.dtype == rows.dtype,
             "queries must be [tokens, n_heads, dim] and the output [tokens, n_heads * vdim]")
    _require_masked_pages(rows, value_pages, queries.dtype, n_kv_heads, dim, vdim)
    _require(vdim <= MASKED_MAX_VALUE_DIM, f"values may have at most {MASKED_MAX_VALUE_DIM} elements per head")
    _require(not (window and chunk), "a window or a chunk, not both")
    _require(page_rows.dtype == torch.int32 and page_rows.dim() == 2 and page_rows.is_contiguous(), "page rows must be int32 [sequences, stride]")
    splits = max(1, min(int(splits), 64)) if staged else 1
    partial = torch.empty((tokens, n_heads, splits, vdim + 2), dtype=torch.float32, device=queries.device) if splits > 1 else None
    library = build.load_library("masked_attention.cu")
    _check(library.tau_masked_attention(
        _code(queries), _pointer(queries), _pointer(rows), _pointer(value_pages), _pointer(out), ctypes.c_longlong(out.stride(0)), _pointer(step.positions), _pointer(step.token_seq),
        _pointer(page_rows), ctypes.c_int(page_rows.shape[1]), ctypes.c_int(PAGE_TOKENS), ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads),
        ctypes.c_int(dim), ctypes.c_int(vdim), ctypes.c_float(scale), ctypes.c_int(window), ctypes.c_int(chunk), ctypes.c_int(1 if sink else 0),
        ctypes.c_float(out_scale), ctypes.c_int(1 if staged else 0), _pointer(distance), ctypes.c_int(1 if sigmoid_weights else 0), _pointer(head_offset),
        _pointer(gate), ctypes.c_longlong(0 if gate is None else gate.stride(0)), ctypes.c_int(1 if gate_per_head else 0), ctypes.c_int(splits), _pointer(partial),
        _stream()), "masked_attention", 2 if splits > 1 else 1)


def gated_rows(values, gate, out) -> None:
    """`out = values * sigmoid(gate)`, element by element; [rows, width] of one dtype, rows any distance apart; `out` may be `values`."""
    _on_device(values, gate, out)
    _require(values.shape == gate.shape == out.shape and values.dim() == 2 and values.dtype == gate.dtype == out.dtype
             and values.stride(1) == gate.stride(1) == out.stride(1) == 1, "values, gate and output must be [rows, width] of one dtype")
    library = build.load_library("masked_attention.cu")
    _check(library.tau_sigmoid_gate(_code(values), _pointer(values), ctypes.c_longlong(values.stride(0)), _pointer(gate), ctypes.c_longlong(gate.stride(0)), _pointer(out),
                                    ctypes.c_longlong(out.stride(0)), ctypes.c_int(values.shape[0]), ctypes.c_int(values.shape[1]), _stream()), "gated_rows")


# ---------------------------------------------------------------------------- a matrix state with a decay per key channel and a bonus
WKV_MAX_KEY_DIM = 512


def token_shift(x, mu, last, step, out, update: bool = True) -> None:
    """`out[s, t] = x[t] + (before[t] - x[t]) * mu[s]` for every vector `mu[s]` (float32 [mixes, width]), `before[t]` being the row of
    the token before in its sequence: `x[t - 1]` inside a run, `last[slot]` (float32 [slots, width], zeros when the sequence starts)
    for a run's first token.  `out` [mixes, tokens, width] of `x`'s dtype.  With `update`, `last[slot]` then becomes the run's last
    row (a second launch, or the same one where every sequence brings one token)."""
    _on_device(x, mu, last, out)
    tokens, width = x.shape
    mixes = mu.shape[0]
    _require(x.is_contiguous() and out.shape == (mixes, tokens, width) and out.dtype == x.dtype and out.is_contiguous(), "the output must be [mixes, tokens, width]")
    _require(mu.dtype == torch.float32 and mu.shape == (mixes, width) and mu.is_contiguous(), "the mixes must be float32 [mixes, width]")
    _require(last.dtype == torch.float32 and last.dim() == 2 and last.shape[1] == width and last.is_contiguous(), "the kept inputs must be float32 [slots, width]")
    single = bool(getattr(step, "all_single", False)) and tokens == step.n_seqs
    library = build.load_library("wkv.cu", ("TAU_KEY_DIM=64",))      # the shift does not depend on the key width
    _check(library.tau_token_shift(_code(x), _pointer(x), _pointer(mu), _pointer(last), _pointer(step.token_seq), _pointer(step.cu_seqlens), _pointer(step.seq_slot),
                                   _pointer(out), ctypes.c_int(tokens), ctypes.c_int(step.n_seqs), ctypes.c_int(width), ctypes.c_int(mixes),
                                   ctypes.c_int(1 if update else 0), ctypes.c_int(1 if single else 0), _stream()), "token_shift", 2 if update and not single else 1)


def tanh_(values) -> None:
    """`values = tanh(values)` in place."""
    _on_device(values)
    _require(values.is_contiguous(), "the values must be contiguous")
    library = build.load_library("wkv.cu", ("TAU_KEY_DIM=64",))
    _check(library.tau_tanh(_code(values), _pointer(values), ctypes.c_longlong(values.numel()), _stream()), "tanh")


def channel_decay(values, offset) -> None:
    """In place on float32 [rows, width]: `exp(-exp(values + offset))`, `offset` float32 [width]."""
    _on_device(values, offset)
    rows, width = values.shape
    _require(values.dtype == torch.float32 and values.is_contiguous(), "the pre-activations must be contiguous float32")
    _f32_vector(offset, width, "the decays' offset")
    library = build.load_library("wkv.cu", ("TAU_KEY_DIM=64",))
    _check(library.tau_channel_decay(_pointer(values), _pointer(offset), ctypes.c_longlong(rows), ctypes.c_int(width), _stream()), "channel_decay")


def wkv(r, k, v, w, bonus, state, cu_seqlens, seq_slot, out, n_heads: int, key_dim: int, value_dim: int) -> None:
    """Per (sequence, head) over the sequence's new tokens: `o = (S + diag(bonus) k v^T)^T r`, then `S <- diag(w) S + k v^T`.
    `r`, `k`, `w` float32 [tokens, n_heads * key_dim], `v` and `out` float32 [tokens, n_heads * value_dim], `bonus` float32
    [n_heads, key_dim], `state` float32 [slots, n_heads * value_dim * key_dim], updated in place."""
    _on_device(r, k, v, w, bonus, state, cu_seqlens, seq_slot, out)
    tokens = r.shape[0]
    for tensor, width, what in ((r, key_dim, "r"), (k, key_dim, "k"), (w, key_dim, "w"), (v, value_dim, "v"), (out, value_dim, "the output")):
        _require(tensor.dtype == torch.float32 and tensor.shape == (tokens, n_heads * width) and tensor.is_contiguous(), f"{what} must be contiguous float32 [tokens, heads * width]")
    _require(bonus.dtype == torch.float32 and bonus.shape == (n_heads, key_dim) and bonus.is_contiguous(), "the bonus must be float32 [heads, key_dim]")
    _require(state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous() and state.shape[1] == n_heads * value_dim * key_dim,
             f"the state must be float32 [slots, {n_heads * value_dim * key_dim}]")
    _require(1 <= key_dim <= WKV_MAX_KEY_DIM, f"key_dim must lie between 1 and {WKV_MAX_KEY_DIM}")
    _int_vector(cu_seqlens, "cu_seqlens")
    _int_vector(seq_slot, "seq_slot")
    n_seqs = seq_slot.numel()
    _require(cu_seqlens.numel() == n_seqs + 1, "one run per sequence")
    library = build.load_library("wkv.cu", (f"TAU_KEY_DIM={key_dim}",))
    _check(library.tau_wkv(_pointer(r), _pointer(k), _pointer(v), _pointer(w), _pointer(bonus), _pointer(state), ctypes.c_longlong(state.stride(0)),
                           _pointer(cu_seqlens), _pointer(seq_slot), _pointer(out), ctypes.c_int(n_seqs), ctypes.c_int(n_heads), ctypes.c_int(value_dim), _stream()), "wkv")


# ---------------------------------------------------------------------------- routed experts
def moe_route(hidden, router, correction, shared_gate_weight, chosen, weights, shared_gate, top: int, softmax: bool = False,
              renormalize: bool = False, logit_bias=None) -> None:
    """Scores the experts of every token in 32-bit and chooses `top` of them: `router` float32 [experts, width];
    scores = sigmoid (or softmax) of `router @ hidden + logit_bias` (float32 [experts] or None); chosen by score + `correction` (float32 [experts] or None), the
    lowest index among equals; `weights` are the chosen scores themselves (divided by their sum with `renormalize`).
    `shared_gate[token] = sigmoid(shared_gate_weight . hidden[token])` where that weight (float32 [width]) is given."""
    _on_device(hidden, router, correction, shared_gate_weight, chosen, weights, shared_gate, logit_bias)
    tokens, width = hidden.shape
    experts = router.shape[0]
    _f32_vector(logit_bias, experts, "the router's bias")
    _require(hidden.is_contiguous() and router.dtype == torch.float32 and router.shape == (experts, width) and router.is_contiguous(),
             "the router must be float32 [experts, width]")
    _f32_vector(correction, experts, "the correction")
    _f32_vector(shared_gate_weight, width, "the shared gate's weight")
    _require(chosen.dtype == torch.int32 and chosen.shape == (tokens, top) and chosen.is_contiguous() and weights.dtype == torch.float32
             and weights.shape == (tokens, top) and weights.is_contiguous(), "chosen must be int32 and weights float32, both [tokens, top]")
    if shared_gate_weight is not None:
        _require(shared_gate is not None and shared_gate.dtype == torch.float32 and shared_gate.numel() == tokens, "one shared gate per token")
    library = build.load_library("moe.cu")
    _check(library.tau_moe_route(_code(hidden), _pointer(hidden), _pointer(router), _pointer(logit_bias), _pointer(correction), _pointer(shared_gate_weight),
                                 _pointer(chosen), _pointer(weights), _pointer(shared_gate), ctypes.c_int(tokens), ctypes.c_int(width),
                                 ctypes.c_int(experts), ctypes.c_int(top), ctypes.c_int(1 if softmax else 0), ctypes.c_int(1 if renormalize else 0),
                                 _stream()), "moe_route")


def moe_gate_up(hidden, gate_up, chosen, inner, interleave: int = 0, input_weights=None) -> None:
    # A pair whose expert number is not below `gate_up.shape[0]` chose an identity expert: its place of `inner` is left unwritten.
    """`inner[token, place] = silu(gate_e @ x) * (up_e @ x)` with `e = chosen[token, place]` and `x = h`, or
    `x = input_weights[token, place] * h` (float32 [tokens, top]; the weight multiplies the two products' 32-bit sums); `gate_up`
    [experts, 2 * I, width] holds each expert's gate rows, then its up rows, or with `interleave` groups of that many gate rows
    each followed by their up rows (what `linear_gated` reads); `inner` [tokens, top, I]."""
    _require(interleave == 0 or inner.shape[2] % interleave == 0, "the interleaved groups must divide the expert's width")
    _on_device(hidden, gate_up, chosen, inner)
    tokens, width = hidden.shape
    top, size = inner.shape[1], inner.shape[2]
    _require(hidden.is_contiguous() and gate_up.is_contiguous() and inner.is_contiguous() and hidden.dtype == gate_up.dtype == inner.dtype,
             "tensors must be contiguous and of one dtype")
    _require(gate_up.shape[1:] == (2 * size, width) and inner.shape[0] == tokens and chosen.shape == (tokens, top) and chosen.dtype == torch.int32
             and chosen.is_contiguous(), "shapes must be [T,W], [E,2I,W], [T,top] -> [T,top,I]")
    if input_weights is not None:
        _on_device(input_weights)
        _require(input_weights.shape == (tokens, top) and input_weights.dtype == torch.float32 and input_weights.is_contiguous(), "input weights must be float32 [tokens, top]")
    library = build.load_library("moe.cu")
    _check(library.tau_moe_gate_up(_code(hidden), _pointer(hidden), _pointer(gate_up), _pointer(chosen), _pointer(input_weights), _pointer(inner), ctypes.c_int(tokens),
                                   ctypes.c_int(width), ctypes.c_int(size), ctypes.c_int(top), ctypes.c_int(interleave), ctypes.c_int(gate_up.shape[0]), _stream()), "moe_gate_up")


def moe_down(inner, down, chosen, weights, shared_out, shared_gate, out, hidden=None) -> None:
    """`out[token] = sum_place weights[token, place] * (down_e @ inner[token, place]) + shared_gate[token] * shared_out[token]`,
    float32 [tokens, width]; `down` [experts, width, I]; `weights` (None: 1), `shared_out` (the activations' dtype) and
    `shared_gate` (float32 [tokens]; None: 1) are optional.  A place whose expert number is not below `down.shape[0]` chose an
    identity expert and adds its weight times `hidden[token]` (what the experts read, [tokens, width]; None: there are no such experts)."""
    _on_device(inner, down, chosen, weights, shared_out, shared_gate, out, hidden)
    if hidden is not None:
        _require(hidden.shape == out.shape and hidden.dtype == inner.dtype and hidden.is_contiguous(), "the experts' input must be [tokens, width]")
    tokens, top, size = inner.shape
    width = down.shape[1]
    _require(inner.is_contiguous() and down.is_contiguous() and inner.dtype == down.dtype and down.shape[2] == size, "down must be [experts, width, I]")
    _require(out.shape == (tokens, width) and out.dtype == torch.float32 and out.is_contiguous(), "the output must be float32 [tokens, width]")
    _require(chosen.shape == (tokens, top) and chosen.dtype == torch.int32 and chosen.is_contiguous() and (weights is None or (weights.shape == (tokens, top)
             and weights.dtype == torch.float32 and weights.is_contiguous())), "chosen and weights must be [tokens, top]")
    if shared_out is not None:
        _require(shared_out.shape == (tokens, width) and shared_out.dtype == inner.dtype and shared_out.is_contiguous(), "the shared output must be [tokens, width]")
    if shared_gate is not None:
        _require(shared_gate.dtype == torch.float32 and shared_gate.numel() == tokens and shared_gate.is_contiguous(), "one shared gate per token")
    library = build.load_library("moe.cu")
    _check(library.tau_moe_down(_code(inner), _pointer(inner), _pointer(down), _pointer(chosen), _pointer(weights), _pointer(shared_out),
                                _pointer(shared_gate), _pointer(out), ctypes.c_int(tokens), ctypes.c_int(width), ctypes.c_int(size), ctypes.c_int(top),
                                _pointer(hidden), ctypes.c_int(down.shape[0]), _stream()), "moe_down")


def moe_sort(chosen, experts: int, offsets, order, position) -> None:
    """Groups the (token, place) pairs of `chosen` [tokens, top] by expert: `order` lists the pairs expert by expert,
    `offsets` [experts + 1] bounds each expert's part of it, `position[pair]` is where a pair went (all int32)."""
    _on_device(chosen, offsets, order, position)
    pairs = chosen.numel()
    _require(chosen.dtype == torch.int32 and chosen.is_contiguous(), "chosen must be contiguous int32")
    for tensor, count, what in ((offsets, experts + 1, "offsets"), (order, pairs, "order"), (position, pairs, "position")):
        _require(tensor.dtype == torch.int32 and tensor.numel() == count and tensor.is_contiguous(), f"{what} must be int32 of {count} elements")
    library = build.load_library("moe.cu")
    _check(library.tau_moe_sort(_pointer(chosen), ctypes.c_int(pairs), ctypes.c_int(experts), _pointer(offsets), _pointer(order), _pointer(position),
                                _stream()), "moe_sort")


def moe_gather(hidden, order, top: int, gathered, input_weights=None) -> None:
    """`gathered[i] = hidden[order[i] // top]`, times `input_weights.view(-1)[order[i]]` (float32, one per pair) if given."""
    _on_device(hidden, order, gathered, input_weights)
    pairs, width = gathered.shape
    _require(hidden.is_contiguous() and gathered.is_contiguous() and hidden.dtype == gathered.dtype and hidden.shape[1] == width
             and order.dtype == torch.int32 and order.numel() == pairs, "gathered must be [pairs, width] of the input's dtype")
    if input_weights is not None:
        _require(input_weights.dtype == torch.float32 and input_weights.numel() == pairs and input_weights.is_contiguous(), "one float32 input weight per pair")
    library = build.load_library("moe.cu")
    _check(library.tau_moe_gather(_code(hidden), _pointer(hidden), _pointer(order), _pointer(input_weights), _pointer(gathered), ctypes.c_int(pairs), ctypes.c_int(width),
                                  ctypes.c_int(top), _stream()), "moe_gather")


def moe_combine(rows, position, weights, shared_out, shared_gate, out, chosen=None, hidden=None, real_experts: int = 0) -> None:
    """`out[token] = sum_place weights[token, place] * rows[position[token, place]] + shared_gate[token] * shared_out[token]`;
    `rows` float32 [pairs, width], `out` float32 [tokens, width]; `weights` None: 1.  With `chosen` ([tokens, top] int32) a place
    whose expert number is not below `real_experts` chose an identity expert: `hidden[token]` stands for its row."""
    _on_device(rows, position, weights, shared_out, shared_gate, out, chosen, hidden)
    if chosen is not None:
        _require(hidden is not None and hidden.shape == out.shape and hidden.is_contiguous() and chosen.dtype == torch.int32 and chosen.numel() == position.numel()
                 and chosen.is_contiguous() and (shared_out is None or shared_out.dtype == hidden.dtype), "identity experts need the experts' input [tokens, width]")
    tokens, width = out.shape
    top = position.numel() // tokens
    _require(rows.dtype == torch.float32 == out.dtype and rows.shape == (tokens * top, width) and rows.is_contiguous() and out.is_contiguous(),
             "rows must be float32 [tokens * top, width]")
    _require(position.dtype == torch.int32 and position.numel() == tokens * top and (weights is None or (weights.dtype == torch.float32 and weights.is_contiguous()
                                                                                            and weights.numel() == tokens * top)),
             "one position and one weight per pair")
    if shared_out is not None:
        _require(shared_out.shape == (tokens, width) and shared_out.is_contiguous(), "the shared output must be [tokens, width]")
    library = build.load_library("moe.cu")
    code = _code(hidden) if chosen is not None else _code(shared_out) if shared_out is not None else 0
    _check(library.tau_moe_combine(code, _pointer(rows), _pointer(position), _pointer(weights),
                                   _pointer(shared_out), _pointer(shared_gate), _pointer(out), ctypes.c_int(tokens), ctypes.c_int(width),
                                   ctypes.c_int(top), _pointer(chosen), _pointer(hidden if chosen is not None else None), ctypes.c_int(real_experts), _stream()), "moe_combine")


# ---------------------------------------------------------------------------- random weights
def random_normal(out: torch.Tensor, key0: int, key1: int, scale: float, shift: float) -> None:
    """Fills `out` (contiguous, float32 or bfloat16) with `shift + scale * n`, n ~ N(0, 1) of the counter-based stream
    `(key0, key1)`; the same bits as `weights.random_init.standard_normals` gives on the host."""
    _on_device(out)
    _require(out.is_contiguous(), "the output must be contiguous")
    library = build.load_library("random_init.cu")
    _check(library.tau_random_normal(_code(out), _pointer(out), ctypes.c_longlong(out.numel()), ctypes.c_uint(key0), ctypes.c_uint(key1),
                                     ctypes.c_float(scale), ctypes.c_float(shift), _stream()), "random_normal")


# ---------------------------------------------------------------------------- selection
_select_scratch = {}


def _scratch_for(logits) -> torch.Tensor:
    library = build.load_library("sampling.cu")
    library.tau_select_scratch_words.restype = ctypes.c_longlong
    words = library.tau_select_scratch_words(ctypes.c_int(logits.shape[0]), ctypes.c_int(logits.shape[1]))
    key = (logits.device, _stream_handle())
    scratch = _select_scratch.get(key)
    if scratch is None or scratch.numel() < words:   # zero once: the tickets at its start; the kernel leaves them at zero
        scratch = _select_scratch[key] = torch.zeros(max(words, 1 << 16), dtype=torch.int32, device=logits.device)
    return scratch


def _check_selection(logits, tokens, valid) -> None:
    _on_device(logits, tokens, valid)
    _require(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(), "logits must be contiguous float32 [rows, vocab]")
    _require(tokens.dtype == torch.int32 and valid.dtype == torch.int32 and tokens.numel() == logits.shape[0] == valid.numel()
             and tokens.is_contiguous() and valid.is_contiguous(), "tokens and valid must be int32 [rows]")


def argmax(logits, tokens, valid) -> None:
    """Greatest logit of each row (NaN left out, highest id among equals); `valid[r] == 0` if the row is all NaN."""
    _check_selection(logits, tokens, valid)
    scratch = _scratch_for(logits)
    library = build.load_library("sampling.cu")
    _check(library.tau_argmax(_pointer(logits), ctypes.c_int(logits.shape[0]), ctypes.c_int(logits.shape[1]), _pointer(scratch),
                              ctypes.c_longlong(scratch.numel()), _pointer(tokens), _pointer(valid), _stream()), "argmax",
           -(-logits.shape[0] // 8192))


def store_words_host(source, pinned_target) -> None:
    """Writes the int32 words of `source` (device, contiguous) into `pinned_target` (page-locked host memory, contiguous, the
    same number of words) from a kernel, in stream order; no copy engine takes part."""
    _require(source.dtype == torch.int32 == pinned_target.dtype and source.is_contiguous() and pinned_target.is_contiguous()
             and source.numel() == pinned_target.numel() and source.is_cuda and not pinned_target.is_cuda and pinned_target.is_pinned(),
             "needs contiguous int32 words on the device and as many in page-locked host memory")
    library = build.load_library("sampling.cu")
    _check(library.tau_store_words_host(_pointer(source), ctypes.c_void_p(pinned_target.data_ptr()), ctypes.c_int(source.numel()), _stream()),
           "store_words_host")


def sample_gumbel(logits, tokens, valid, inverse_temperature: float, seed: int, request_ids, token_indices) -> None:
    _check_selection(logits, tokens, valid)
    _on_device(request_ids, token_indices)
    _int_vector(request_ids, "request ids")
    _int_vector(token_indices, "token indices")
    _require(request_ids.numel() == logits.shape[0] == token_indices.numel(), "one request id and token index per row")
    scratch = _scratch_for(logits)
    library = build.load_library("sampling.cu")
    _check(library.tau_sample_gumbel(_pointer(logits), ctypes.c_int(logits.shape[0]), ctypes.c_int(logits.shape[1]), _pointer(scratch),
                                     ctypes.c_longlong(scratch.numel()), _pointer(tokens), _pointer(valid),
                                     ctypes.c_float(inverse_temperature), ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF),
                                     _pointer(request_ids), _pointer(token_indices), _stream()), "sample_gumbel",
           -(-logits.shape[0] // 8192))
