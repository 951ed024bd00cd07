"""Plain torch statement of what each CUDA kernel computes, with the same call signature.

Used in two ways: on the GPU each kernel is compared with its function here, at sizes
other than the engine's; on the CPU these functions stand in for the kernels so that the
engine's host logic (packing, pages, slots, schedule) can be tested without a GPU.  They are
test code: the library never imports them and has no CPU path of its own.  Arithmetic is
32-bit with a rounding to the tensor's dtype wherever the kernel stores.
"""
from __future__ import annotations

import numpy as np
import torch

PAGE_TOKENS = 64


def _wide(tensor):
    return tensor.to(torch.float32)


def embedding(tokens, table, out):
    out.copy_(table[tokens.long()])


def rms_norm(values, weight, eps, out, rows=None, branch=None):
    source = _wide(values)
    if branch is not None:
        source = _wide((source + _wide(branch)).to(values.dtype))
    if rows is not None:
        source = source[rows.long()]
    inverse = torch.rsqrt(source.pow(2).mean(dim=-1, keepdim=True) + eps)
    out.copy_((source * inverse * weight).to(out.dtype))


def add_rms_norm(branch, residual, weight, eps, out):
    residual.copy_((_wide(residual) + _wide(branch)).to(residual.dtype))
    rms_norm(residual, weight, eps, out)


def silu_mul(stacked, out):
    width = out.shape[-1]
    gate, up = _wide(stacked[:, :width]), _wide(stacked[:, width:])
    out.copy_((gate / (1.0 + torch.exp(-gate)) * up).to(out.dtype))


def linear(values, weight, bias, out):
    result = _wide(values).double() @ _wide(weight).double().t()
    if bias is not None:
        result = result + bias.double()
    out.copy_(result.to(out.dtype))


gemm_simt = linear
GATE_GROUP = 8


def gated_fits(in_features, out_features, dtype):
    return False     # the host-logic tests keep the product and the activation apart


def linear_gated(values, weight, out):
    """Rows of `weight`: groups of 8 gate rows followed by their 8 up rows."""
    width = weight.shape[1]
    grouped = weight.view(-1, 2, GATE_GROUP, width)
    gate, up = grouped[:, 0].reshape(-1, width), grouped[:, 1].reshape(-1, width)
    g = torch.empty(values.shape[0], gate.shape[0], dtype=values.dtype)
    u = torch.empty_like(g)
    linear(values, gate, None, g)
    linear(values, up, None, u)
    silu_mul(torch.cat([g, u], dim=1), out)


def _page_offsets(page_rows, token_seq, positions):
    pages = page_rows[token_seq.long(), (positions // PAGE_TOKENS).long()].long()
    return pages, (positions % PAGE_TOKENS).long()


def attention_prepare(projected, queries, keys, values, write_cache, q_weight, k_weight, eps, cos, sin, rotary_dim, positions,
                      token_seq, page_rows, n_heads, n_kv_heads, head_dim):
    tokens = projected.shape[0]
    dtype = projected.dtype
    q_width, kv_width = n_heads * head_dim, n_kv_heads * head_dim

    def prepare(block, heads, weight):
        block = _wide(block).view(tokens, heads, head_dim)
        if weight is not None:
            inverse = torch.rsqrt(block.pow(2).mean(dim=-1, keepdim=True) + eps)
            block = _wide((block * inverse * weight).to(dtype))
        if rotary_dim:
            half = rotary_dim // 2
            c = cos[positions.long()][:, None, :]
            s = sin[positions.long()][:, None, :]
            first, second = block[..., :half], block[..., half:rotary_dim]
            rotated = torch.cat([first * c - second * s, second * c + first * s, block[..., rotary_dim:]], dim=-1)
            block = rotated
        return block.to(dtype)

    queries.copy_(prepare(projected[:, :q_width], n_heads, q_weight).view(tokens, q_width))
    if write_cache:
        new_keys = prepare(projected[:, q_width : q_width + kv_width], n_kv_heads, k_weight)
        new_values = projected[:, q_width + kv_width : q_width + 2 * kv_width].reshape(tokens, n_kv_heads, head_dim)
        pages, places = _page_offsets(page_rows, token_seq, positions)
        keys[pages, :, places, :] = new_keys
        values[pages, :, places, :] = new_values


def attention_generic(queries, keys, values, out, positions, token_seq, page_rows, n_heads, n_kv_heads, head_dim, scale, window):
    tokens = queries.shape[0]
    group = n_heads // n_kv_heads
    q = _wide(queries).view(tokens, n_heads, head_dim)
    result = torch.empty_like(q)
    for token in range(tokens):
        position = int(positions[token])
        first = max(0, position - window + 1) if window else 0
        span = torch.arange(first, position + 1)
        pages = page_rows[int(token_seq[token]), (span // PAGE_TOKENS).long()].long()
        places = (span % PAGE_TOKENS).long()
        k = _wide(keys[pages, :, places, :])      # [span, kv, d]
        v = _wide(values[pages, :, places, :])
        for head in range(n_heads):
            scores = (k[:, head // group, :] @ q[token, head]) * scale
            weights = torch.softmax(scores, dim=0)
            result[token, head] = weights @ v[:, head // group, :]
    out.copy_(result.view(tokens, n_heads * head_dim).to(out.dtype))


def decode_splits(n_seqs, max_len, kv_blocks=8):
    return 1


def attention_decode_fused(*args, **kwargs):
    return False     # the plain statement keeps prepare and attention apart


def attention(queries, keys, values, out, step, page_rows, n_heads, n_kv_heads, head_dim, scale, window):
    attention_generic(queries, keys, values, out, step.positions, step.token_seq, page_rows, n_heads, n_kv_heads, head_dim, scale, window)


def _order_keys(values: np.ndarray):
    bits = values.astype(np.float32).view(np.uint32).astype(np.int64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    keys = np.where(bits & 0x80000000, bits ^ 0xFFFFFFFF, bits ^ 0x80000000)
    return keys, nan


def argmax_row(values: np.ndarray):
    """(token, valid): greatest by total order, NaN left out, highest index among equals."""
    keys, nan = _order_keys(values)
    if nan.all():
        return 0, 0
    keys = np.where(nan, -1, keys)
    best = keys.max()
    return int(np.nonzero(keys == best)[0][-1]), 1


def argmax(logits, tokens, valid):
    for row in range(logits.shape[0]):
        token, ok = argmax_row(logits[row].cpu().numpy())
        tokens[row], valid[row] = token, ok


def philox_first_word(c0, c1, c2, c3, k0, k1):
    """Philox4x32-10 on numpy uint64 arrays holding 32-bit words; returns the first output word."""
    mask = np.uint64(0xFFFFFFFF)
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) & mask for c in (c0, c1, c2, c3))
    k0, k1 = np.uint64(k0), np.uint64(k1)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & mask, lo1, (hi0 ^ c3 ^ k1) & mask, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return c0


def gumbel_scores(row: np.ndarray, inverse_temperature, seed, request, token_index):
    vocab = row.shape[0]
    zeros = np.zeros(vocab, dtype=np.uint64)
    word = philox_first_word(np.arange(vocab, dtype=np.uint64), zeros + np.uint64(token_index), zeros + np.uint64(request), zeros,
                             seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    u = ((word >> np.uint64(8)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return (row.astype(np.float32) * np.float32(inverse_temperature) - np.log(-np.log(u))).astype(np.float32)


def sample_gumbel(logits, tokens, valid, inverse_temperature, seed, request_ids, token_indices):
    for row in range(logits.shape[0]):
        scores = gumbel_scores(logits[row].cpu().numpy(), inverse_temperature, seed, int(request_ids[row]), int(token_indices[row]))
        token, ok = argmax_row(scores)
        tokens[row], valid[row] = token, ok


ALL = ("embedding", "rms_norm", "add_rms_norm", "silu_mul", "linear", "gemm_simt", "gated_fits", "linear_gated", "attention_prepare", "attention_generic",
       "attention", "attention_decode_fused", "decode_splits", "argmax", "sample_gumbel")


def install(monkeypatch):
    """Replaces the kernel functions by the functions of this file (CPU tests of host logic only)."""
    from tau_rs_b200.csrc import kernels

    module = __import__(__name__)
    for name in ALL:
        monkeypatch.setattr(kernels, name, getattr(module, name))
