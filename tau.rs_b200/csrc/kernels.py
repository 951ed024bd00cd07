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
}
_timing = None     # while timing: [last event, [(class, event after the launch), ...]]


def start_timing() -> None:
    """From now on an event follows every launch of this library on the current stream; `take_timing` reads them.
    Meant for steps that run outside a captured graph."""
    global _timing
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
        _timing[1].append((_CLASS_OF.get(what, "other"), event))
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
def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    _on_device(tokens, table, out)
    _int_vector(tokens, "token ids")
    _require(table.dtype == out.dtype and table.is_contiguous() and out.is_contiguous(), "table and output must match")
    _require(out.shape == (tokens.shape[0], table.shape[1]), "output must be [tokens, width]")
    library = build.load_library("elementwise.cu")
    _check(library.tau_embedding(_code(table), _pointer(tokens), _pointer(table), _pointer(out), ctypes.c_int(tokens.shape[0]),
                                 ctypes.c_int(table.shape[1]), ctypes.c_int(table.shape[0]), _stream()), "embedding")


def rms_norm(values, weight, eps: float, out, rows=None, branch=None) -> None:
    """`out[i] = norm(round(values[r] + branch[r])) * weight`, `r = rows[i]` or `i`; `values` is not changed."""
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


def add_rms_norm(branch, residual, weight, eps: float, out) -> None:
    """`residual = round(residual + branch)` in place; `out = norm(residual) * weight`."""
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


def silu_mul(stacked, out) -> None:
    """`out[r, c] = silu(stacked[r, c]) * stacked[r, width + c]`."""
    _on_device(stacked, out)
    width = out.shape[-1]
    _require(stacked.shape[-1] == 2 * width and stacked.shape[0] == out.shape[0] and stacked.dtype == out.dtype,
             "input must be [rows, 2 * width] and output [rows, width]")
    _require(stacked.is_contiguous() and out.is_contiguous(), "tensors must be contiguous")
    library = build.load_library("elementwise.cu")
    _check(library.tau_silu_mul(_code(out), _pointer(stacked), _pointer(out), ctypes.c_longlong(out.shape[0]), ctypes.c_int(width),
                                _stream()), "silu_mul")


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
                      scale: float, window: int) -> None:
    """bfloat16 causal attention of runs of new tokens (`cu_seqlens` bounds them, `seq_start` positions were cached before)."""
    _on_device(queries, keys, values, out, cu_seqlens, seq_start, page_rows)
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
        ctypes.c_int(n_kv_heads), ctypes.c_float(scale), ctypes.c_int(window), _stream()), "attention_prefill")


_prefill_schedule = {}   # (device, stream) -> the two counters by which the blocks of the tensor-core prefill kernel share out its tiles


def attention_prefill_tc(queries, keys, values, out, cu_seqlens, seq_start, page_rows, n_heads: int, n_kv_heads: int, head_dim: int,
                         scale: float, window: int) -> None:
    """The same as `attention_prefill` on the tcgen05 tensor cores (accumulators in tensor memory); head sizes 64 and 128."""
    _on_device(queries, keys, values, out, cu_seqlens, seq_start, page_rows)
    tokens = queries.shape[0]
    n_seqs = seq_start.numel()
    _require(head_dim in (64, 128), "the tensor-core prefill kernel serves head sizes 64 and 128")
    _require(queries.dtype == torch.bfloat16 == out.dtype == keys.dtype == values.dtype, "the tensor-core prefill kernel is bfloat16 only")
    _require(queries.shape == (tokens, n_heads * head_dim) and out.shape == queries.shape and queries.is_contiguous() and out.is_contiguous(),
             "queries and output must be [tokens, n_heads * head_dim]")
    _require(n_heads % n_kv_heads == 0, "n_heads must be a multiple of n_kv_heads")
    _require(keys.shape[1:] == (n_kv_heads, PAGE_TOKENS, head_dim) and keys.is_contiguous() and values.is_contiguous()
             and values.shape == keys.shape, "cache pages must be [pages, n_kv_heads, 64, head_dim]")
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
        ctypes.c_int(tokens), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_float(scale), ctypes.c_int(window),
        _pointer(schedule), _stream()),
        "attention_prefill_tc")


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
