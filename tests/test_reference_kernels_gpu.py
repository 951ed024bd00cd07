"""This library's kernels against the reference's own, on the same inputs.

taurs-ai/tau.rs cannot be built here (a Rust workspace, its dense Qwen3 layer math in a crate that is not on disk), but
four of its CUDA sources compile on their own and export C launchers; `baseline/build_ref.py` builds them unchanged
into `baseline/_ref/`.  They are the only code of the reference that can produce a number on this machine, so these
tests are where a reading of the reference is checked against the reference's output: which elements a rotation
pairs, that the per-head norm comes before the rotation, which KV head a query head reads, how split contexts merge,
which token a greedy selection picks, where a residual sum is rounded.  Its norms scale by `1 + w`
(crates/cuda-kernels/src/kernels/decode_attention.cu:152, centered_rms_norm.cu), dense Qwen3's by `w`, so the reference
gets `w - 1`, which is exact for the weights used here.  The tests are skipped where the binaries are absent.
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))

import reference_kernels  # noqa: E402
from tau_rs_b200.csrc import kernels  # noqa: E402
from test_kernels_gpu import adversarial_rows  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not reference_kernels.available(), reason="baseline/_ref holds no built reference kernels")]
DEVICE = "cuda"
BF16 = torch.bfloat16


def close(found, wanted, tolerance):
    error = float((found.double().cpu() - wanted.double().cpu()).abs().max() / wanted.double().abs().max().clamp_min(1e-30))
    assert error < tolerance, error


def reference_argmax(row: torch.Tensor):
    scratch = torch.empty(max(3 * (row.numel() // 1024 + 1), 16), dtype=torch.int32, device=DEVICE)
    result = torch.full((2,), -7, dtype=torch.int32, device=DEVICE)
    reference_kernels.greedy_argmax(row, scratch, result)
    token, valid = result.tolist()
    return token, valid


def test_greedy_selection_picks_the_reference_token():
    """The reference's adversarial cases (crates/engine/src/generation/greedy/tests.rs:18-48) and random bit patterns of
    its lengths (:86-123), row by row through `tau_launch_greedy_argmax` and all at once through this library's kernel."""
    for row in adversarial_rows():
        logits = torch.tensor([row], dtype=torch.float32, device=DEVICE)
        tokens = torch.full((1,), -7, dtype=torch.int32, device=DEVICE)
        valid = torch.full((1,), -7, dtype=torch.int32, device=DEVICE)
        kernels.argmax(logits, tokens, valid)
        token, ok = reference_argmax(logits[0].contiguous())
        assert int(valid[0]) == ok, row
        assert not ok or int(tokens[0]) == token, row
    for vocab in (1, 31, 32, 33, 255, 256, 257, 1023, 1024, 1025, 248320):
        rng = np.random.default_rng(vocab)
        bits = rng.integers(0, 2 ** 32, size=(4, vocab), dtype=np.uint64).astype(np.uint32)
        bits[1, :] = bits[1, 0]
        bits[2, :] = 0xFFC00000
        bits[3, vocab // 2:] = 0x7F800000
        logits = torch.from_numpy(bits.view(np.float32).copy()).to(DEVICE)
        tokens = torch.empty(4, dtype=torch.int32, device=DEVICE)
        valid = torch.empty(4, dtype=torch.int32, device=DEVICE)
        kernels.argmax(logits, tokens, valid)
        for row in range(4):
            token, ok = reference_argmax(logits[row].contiguous())
            assert int(valid[row]) == ok, (vocab, row)
            assert not ok or int(tokens[row]) == token, (vocab, row)


@pytest.mark.parametrize("dtype", [torch.float32, BF16])
@pytest.mark.parametrize("rows,columns", [(1, 16), (7, 224), (3, 12288), (130, 1000)])
def test_the_activation_of_the_feed_forward(dtype, rows, columns):
    generator = torch.Generator().manual_seed(rows * columns)
    stacked = (torch.randn(rows, 2 * columns, generator=generator) * 3).to(dtype).to(DEVICE)
    wanted = torch.empty(rows, columns, dtype=dtype, device=DEVICE)
    found = torch.empty_like(wanted)
    reference_kernels.silu_and_mul(stacked, wanted)
    kernels.silu_mul(stacked, found)
    close(found, wanted, 1e-6 if dtype == torch.float32 else 4e-3)   # at most the last place of a bfloat16 value


def norm_weights(width, seed):
    """Weights `w` near one that bfloat16 holds, and `w - 1`, which it then holds as well."""
    weight = (1 + 0.1 * torch.randn(width, generator=torch.Generator().manual_seed(seed))).to(BF16)
    centered = (weight.float() - 1.0).to(BF16)
    assert torch.equal(centered.float() + 1.0, weight.float())
    return weight.float().to(DEVICE), centered.to(DEVICE)


@pytest.mark.parametrize("rows,width,eps", [(5, 128, 1e-6), (3, 1000, 1e-5), (9, 4096, 1e-6), (2, 5120, 1e-6), (4, 2560, 1e-6)])
def test_norms_and_the_rounded_residual_sum(rows, width, eps):
    generator = torch.Generator().manual_seed(width)
    values = (torch.randn(rows, width, generator=generator) * 2).to(BF16).to(DEVICE)
    branch = torch.randn(rows, width, generator=generator).to(BF16).to(DEVICE)
    weight, centered = norm_weights(width, width + 1)
    wanted = torch.empty_like(values)
    found = torch.empty_like(values)
    reference_kernels.centered_rms_norm(values, centered, eps, wanted)
    kernels.rms_norm(values, weight, eps, found)
    close(found, wanted, 4e-3)
    wanted_sum = torch.empty_like(values)
    reference_kernels.fused_residual_rms_norm(values, branch, centered, wanted_sum, wanted, eps)
    residual = values.clone()
    kernels.add_rms_norm(branch, residual, weight, eps, found)
    assert torch.equal(residual, wanted_sum)          # the sum is rounded to bfloat16 once, before the norm reads it
    close(found, wanted, 4e-3)


@pytest.mark.parametrize("heads,kv_heads,dim,position,theta", [(32, 8, 128, 300, 1e6), (6, 2, 64, 700, 1e4), (8, 1, 32, 63, 1e6), (4, 4, 16, 64, 1e4)])
def test_one_decoded_token_through_prepare_attention_and_merge(heads, kv_heads, dim, position, theta):
    """One token at `position` over a history of random keys and values: the reference's `attention_prepare`, `attention`
    and `combine_attention` (decode_attention.cu:120-181,186-278) on a `[kv_heads, capacity, dim]` cache whose tail is
    NaN, against this library's prepare and decode kernels, separate and fused, on a paged cache that holds the same rows
    on shuffled pages."""
    from tau_rs_b200.config import PositionSpec
    from tau_rs_b200.parts.registry import build

    capacity = 1024
    generator = torch.Generator().manual_seed(position)
    eps = 1e-6
    history_k = torch.randn(kv_heads, position, dim, generator=generator).to(BF16)
    history_v = torch.randn(kv_heads, position, dim, generator=generator).to(BF16)
    history_k[kv_heads - 1, position // 3] *= 6.0          # one far key that some head's softmax leans on
    projected = torch.randn(1, (heads + 2 * kv_heads) * dim, generator=generator).to(BF16).to(DEVICE)
    q_weight, q_centered = norm_weights(dim, 5)
    k_weight, k_centered = norm_weights(dim, 6)
    rope = build("position", PositionSpec(rotary_dim=dim, theta=theta, max_positions=capacity), device=torch.device(DEVICE))
    rope.finalize_weights()

    # ---- the reference
    query_gate = torch.zeros(heads, 2 * dim, dtype=BF16, device=DEVICE)
    query_gate[:, :dim] = projected[0, : heads * dim].view(heads, dim)
    key = projected[0, heads * dim : (heads + kv_heads) * dim].view(kv_heads, dim).contiguous()
    value = projected[0, (heads + kv_heads) * dim :].view(kv_heads, dim).contiguous()
    cache_k = torch.full((kv_heads, capacity, dim), float("nan"), dtype=BF16, device=DEVICE)
    cache_v = torch.full((kv_heads, capacity, dim), float("nan"), dtype=BF16, device=DEVICE)
    cache_k[:, :position] = history_k.to(DEVICE)
    cache_v[:, :position] = history_v.to(DEVICE)
    meta = torch.tensor([0, position], dtype=torch.int32, device=DEVICE)
    wanted_q = torch.empty(heads * dim, dtype=BF16, device=DEVICE)
    reference_kernels.decode_attention_prepare(query_gate, key, value, q_centered, k_centered, rope.cos, rope.sin, wanted_q, cache_k, cache_v,
                                               meta, heads, kv_heads, dim, capacity, dim, eps)
    wanted = {}
    for block_size in (64, 256):
        workspace = torch.empty(heads * (capacity // block_size) * (dim + 2), dtype=torch.float32, device=DEVICE)
        wanted[block_size] = torch.empty(heads * dim, dtype=BF16, device=DEVICE)
        reference_kernels.decode_attention(wanted_q, cache_k, cache_v, wanted[block_size], meta, workspace, heads, kv_heads, dim, capacity, block_size)
    close(wanted[64], wanted[256], 1e-2)
    assert torch.equal(cache_v[:, position], value)

    # ---- this library, on pages
    n_pages = capacity // 64
    order = torch.randperm(n_pages + 3, generator=generator)[:n_pages].to(torch.int32)
    keys = torch.full((n_pages + 3, kv_heads, 64, dim), float("nan"), dtype=BF16, device=DEVICE)
    values = torch.full((n_pages + 3, kv_heads, 64, dim), float("nan"), dtype=BF16, device=DEVICE)
    for index in range(position):
        keys[order[index // 64], :, index % 64] = history_k[:, index].to(DEVICE)
        values[order[index // 64], :, index % 64] = history_v[:, index].to(DEVICE)
    page_rows = order.view(1, n_pages).to(DEVICE).contiguous()
    positions = torch.tensor([position], dtype=torch.int32, device=DEVICE)
    token_seq = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    seq_len = torch.tensor([position + 1], dtype=torch.int32, device=DEVICE)
    found_q = torch.empty(1, heads * dim, dtype=BF16, device=DEVICE)
    separate_k, separate_v = keys.clone(), values.clone()
    kernels.attention_prepare(projected, found_q, separate_k, separate_v, True, q_weight, k_weight, eps, rope.cos, rope.sin, dim, positions,
                              token_seq, page_rows, heads, kv_heads, dim)
    close(found_q.view(-1), wanted_q, 1e-2)
    page, place = int(order[position // 64]), position % 64
    close(separate_k[page, :, place], cache_k[:, position], 1e-2)
    assert torch.equal(separate_v[page, :, place], value)
    for splits in (1, 4, 16):
        found = torch.full((1, heads * dim), float("nan"), dtype=BF16, device=DEVICE)
        kernels.attention_decode(found_q, separate_k, separate_v, found, seq_len, page_rows, heads, kv_heads, dim, dim ** -0.5, 0, splits)
        close(found.view(-1), wanted[64], 1e-2)
        fused_k, fused_v = keys.clone(), values.clone()
        found = torch.full((1, heads * dim), float("nan"), dtype=BF16, device=DEVICE)
        kernels.attention_decode(None, fused_k, fused_v, found, seq_len, page_rows, heads, kv_heads, dim, dim ** -0.5, 0, splits,
                                 prepare=(projected, q_weight, k_weight, eps, rope.cos, rope.sin, dim, True))
        close(found.view(-1), wanted[64], 1e-2)
        close(fused_k[page, :, place], cache_k[:, position], 1e-2)
        assert torch.equal(fused_v[page, :, place], value)
    # Head by head, so that a query head that read another KV head cannot hide behind a larger head.
    per_head_found, per_head_wanted = found.view(heads, dim), wanted[64].view(heads, dim)
    for head in range(heads):
        close(per_head_found[head], per_head_wanted[head], 2e-2)
