"""The reference's generic CUDA kernels, called through their own C launchers (built by `build_ref.py`).

Nothing of this library is loaded here: the shared objects under `baseline/_ref/` hold only taurs-ai/tau.rs's
sources (crates/cuda-kernels/src/kernels/{greedy_argmax,silu_and_mul,decode_attention,centered_rms_norm}.cu).
torch serves as the owner of device memory and of the stream.  Every wrapper checks what the launcher itself
would refuse, and the sizes that its kernels assume without checking, before it launches.
"""
from __future__ import annotations

import ctypes
import os

import torch

_REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_NAMES = ("greedy_argmax", "silu_and_mul", "decode_attention", "centered_rms_norm")
_loaded = {}


def available() -> bool:
    return all(os.path.isfile(os.path.join(_REF, name + ".so")) for name in _NAMES)


def _library(name: str) -> ctypes.CDLL:
    if name not in _loaded:
        _loaded[name] = ctypes.CDLL(os.path.join(_REF, name + ".so"))
    return _loaded[name]


def _p(tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(tensor.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _code(tensor) -> int:
    return {torch.float32: 0, torch.bfloat16: 1}[tensor.dtype]


def _ok(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"the reference's {what} returned {status}")


def _device(*tensors) -> None:
    for tensor in tensors:
        assert tensor.is_cuda and tensor.is_contiguous(), "contiguous CUDA tensors only"


def greedy_argmax(logits: torch.Tensor, scratch: torch.Tensor, result: torch.Tensor) -> None:
    """`tau_launch_greedy_argmax` (greedy_argmax.cu:101-117): `logits` `[V]` float32 or bfloat16; `result` two uint32
    words `[token, valid]`; `scratch` at least `tau_greedy_argmax_workspace_words(V)` words."""
    _device(logits, scratch, result)
    library = _library("greedy_argmax")
    library.tau_greedy_argmax_workspace_words.restype = ctypes.c_size_t
    count = logits.numel()
    words = library.tau_greedy_argmax_workspace_words(ctypes.c_uint(count))
    assert logits.dim() == 1 and count > 0 and scratch.dtype == torch.int32 and scratch.numel() >= words
    assert result.dtype == torch.int32 and result.numel() >= 2
    _ok(library.tau_launch_greedy_argmax(_p(logits), ctypes.c_int(_code(logits)), ctypes.c_uint(count), _p(scratch),
                                         ctypes.c_size_t(scratch.numel()), _p(result), _stream()), "greedy argmax")


def silu_and_mul(stacked: torch.Tensor, out: torch.Tensor) -> None:
    """`tau_launch_silu_and_mul` (silu_and_mul.cu:90-132): `out[r, c] = silu(stacked[r, c]) * stacked[r, C + c]`."""
    _device(stacked, out)
    rows, columns = out.shape
    assert stacked.shape == (rows, 2 * columns) and stacked.dtype == out.dtype
    _ok(_library("silu_and_mul").tau_launch_silu_and_mul(_p(stacked), _p(out), ctypes.c_int(rows), ctypes.c_int(columns),
                                                         ctypes.c_int(_code(out)), _stream()), "silu_and_mul")


def centered_rms_norm(values: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """`tau_launch_centered_rms_norm` (centered_rms_norm.cu:511-517): `x * rsqrt(mean(x^2) + eps) * (1 + weight)`; the
    weight has the values' dtype."""
    _device(values, weight, out)
    rows, columns = values.shape
    assert out.shape == values.shape and weight.shape == (columns,) and values.dtype == weight.dtype == out.dtype
    _ok(_library("centered_rms_norm").tau_launch_centered_rms_norm(_p(values), _p(weight), _p(out), ctypes.c_int(rows), ctypes.c_int(columns),
                                                                   ctypes.c_float(eps), ctypes.c_int(_code(values)), _stream()), "centered rms norm")


def fused_residual_rms_norm(values, branch, weight, residual_out, out, eps: float) -> None:
    """`tau_launch_fused_residual_rms_norm` (centered_rms_norm.cu:545-565): `residual_out = round(values + branch)`,
    `out = norm(residual_out) * (1 + weight)`; no input is changed, the outputs are distinct buffers."""
    _device(values, branch, weight, residual_out, out)
    rows, columns = values.shape
    assert branch.shape == residual_out.shape == out.shape == values.shape and weight.shape == (columns,)
    assert values.dtype == branch.dtype == weight.dtype == residual_out.dtype == out.dtype
    assert len({values.data_ptr(), branch.data_ptr(), residual_out.data_ptr(), out.data_ptr()}) == 4
    _ok(_library("centered_rms_norm").tau_launch_fused_residual_rms_norm(
        _p(values), _p(branch), _p(weight), _p(residual_out), _p(out), ctypes.c_int(rows), ctypes.c_int(columns), ctypes.c_float(eps),
        ctypes.c_int(_code(values)), _stream(), ctypes.c_int(16)), "fused residual rms norm")


def _attention_shapes(heads: int, kv_heads: int, dim: int, capacity: int) -> None:
    assert heads > 0 and kv_heads > 0 and heads % kv_heads == 0 and 0 < dim <= 256 and 0 < capacity <= 8192


def decode_attention_prepare(query_gate, key, value, query_weight, key_weight, cos, sin, query_out, cached_key, cached_value, meta,
                             heads: int, kv_heads: int, dim: int, capacity: int, rotary_dim: int, eps: float, position: int = None) -> None:
    """`tau_launch_decode_attention_prepare` (decode_attention.cu:307-345) with 32-bit rotation tables and the
    position-major cache: one token at position `meta[1]`; `query_gate` `[heads, 2 dim]` (the query, then a gate that is
    not read), `key`/`value` `[kv_heads, dim]`, norm weights `[dim]` scaling by `1 + w`, tables `[positions, rotary_dim / 2]`
    float32, caches `[kv_heads, capacity, dim]`."""
    _device(query_gate, key, value, query_weight, key_weight, cos, sin, query_out, cached_key, cached_value, meta)
    _attention_shapes(heads, kv_heads, dim, capacity)
    bf16 = torch.bfloat16
    assert query_gate.shape == (heads, 2 * dim) and key.shape == value.shape == (kv_heads, dim) and query_out.numel() == heads * dim
    assert all(t.dtype == bf16 for t in (query_gate, key, value, query_weight, key_weight, query_out, cached_key, cached_value))
    assert query_weight.numel() == key_weight.numel() == dim and cached_key.shape == cached_value.shape == (kv_heads, capacity, dim)
    assert 0 < rotary_dim <= dim and rotary_dim % 2 == 0 and cos.dtype == sin.dtype == torch.float32 and cos.shape == sin.shape
    assert meta.dtype == torch.int32 and meta.numel() == 2
    position = int(meta[1]) if position is None else position     # a caller that times the launch names the position itself
    assert 0 <= position < capacity and position < cos.shape[0] and cos.shape[1] == rotary_dim // 2 and eps > 0
    _ok(_library("decode_attention").tau_launch_decode_attention_prepare(
        _p(query_gate), _p(key), _p(value), _p(query_weight), _p(key_weight), _p(cos), _p(sin), _p(query_out), _p(cached_key), _p(cached_value),
        _p(meta), ctypes.c_int(heads), ctypes.c_int(kv_heads), ctypes.c_int(dim), ctypes.c_int(capacity), ctypes.c_int(rotary_dim),
        ctypes.c_int(0), ctypes.c_int(1), ctypes.c_float(eps), ctypes.c_float(eps), _stream()), "attention prepare")


def decode_attention(query, cached_key, cached_value, out, meta, workspace, heads: int, kv_heads: int, dim: int, capacity: int,
                     block_size: int, position: int = None) -> None:
    """`tau_launch_decode_attention` (decode_attention.cu:348-365) with 32-bit products: one query token at position
    `meta[1]` over the positions `0 .. meta[1]` of the caches; the context is cut into tiles of `block_size` positions
    whose records `(max, sum, context)` a second kernel merges.  `workspace`: `heads * ceil(capacity / block_size) *
    (dim + 2)` floats."""
    _device(query, cached_key, cached_value, out, meta, workspace)
    _attention_shapes(heads, kv_heads, dim, capacity)
    assert block_size in (32, 64, 128, 256)
    splits = -(-capacity // block_size)
    assert splits <= 256 and workspace.dtype == torch.float32 and workspace.numel() >= heads * splits * (dim + 2)
    assert query.numel() == out.numel() == heads * dim and query.dtype == out.dtype == cached_key.dtype == cached_value.dtype == torch.bfloat16
    assert cached_key.shape == cached_value.shape == (kv_heads, capacity, dim) and meta.dtype == torch.int32 and meta.numel() == 2
    assert 0 <= (int(meta[1]) if position is None else position) < capacity
    _ok(_library("decode_attention").tau_launch_decode_attention(
        _p(query), _p(cached_key), _p(cached_value), _p(out), _p(meta), _p(workspace), ctypes.c_int(heads), ctypes.c_int(kv_heads),
        ctypes.c_int(dim), ctypes.c_int(capacity), ctypes.c_int(0), ctypes.c_int(block_size), ctypes.c_int(0), _stream()), "decode attention")
