"""Each CUDA kernel alone against its plain statement, at sizes other than the engine's."""
import numpy as np
import pytest
import torch

import plain_kernels
from tau_rs_b200.csrc import kernels

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
DTYPES = [torch.float32, torch.bfloat16]
# Relative to the largest expected magnitude; bfloat16 stores keep 8 bits.
TOLERANCE = {torch.float32: 2e-5, torch.bfloat16: 1e-2}


def close(found, wanted, dtype, scale=1.0):
    found, wanted = found.double().cpu(), wanted.double().cpu()
    error = float((found - wanted).abs().max() / wanted.abs().max().clamp_min(1e-30))
    assert error < TOLERANCE[dtype] * scale, error


def randn(*shape, dtype, seed, scale=1.0):
    generator = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=generator) * scale).to(dtype).to(DEVICE)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,vocab", [(7, 11), (96, 500), (1000, 333)])
def test_embedding(dtype, width, vocab):
    table = randn(vocab, width, dtype=dtype, seed=1)
    tokens = torch.tensor([0, vocab - 1, 3, 3, vocab // 2], dtype=torch.int32, device=DEVICE)
    out = torch.empty(5, width, dtype=dtype, device=DEVICE)
    kernels.embedding(tokens, table, out)
    assert torch.equal(out, table[tokens.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,eps", [(1, 16, 1e-6), (5, 97, 1e-5), (3, 1000, 1e-3), (2, 4100, 1e-6), (9, 4096, 1e-6), (2, 8192, 1e-5), (2, 12288, 1e-6)])
def test_rms_norm(dtype, rows, width, eps):
    values = randn(rows, width, dtype=dtype, seed=2, scale=3.0)
    branch = randn(rows, width, dtype=dtype, seed=3)
    weight = (1 + 0.1 * torch.randn(width, generator=torch.Generator().manual_seed(4))).to(DEVICE)
    for use_branch in (False, True):
        for picked in (None, torch.tensor([rows - 1, 0, rows - 1], dtype=torch.int32, device=DEVICE)):
            count = rows if picked is None else 3
            found = torch.empty(count, width, dtype=dtype, device=DEVICE)
            wanted = torch.empty(count, width, dtype=dtype)
            before = values.clone()
            kernels.rms_norm(values, weight, eps, found, picked, branch if use_branch else None)
            plain_kernels.rms_norm(values.cpu(), weight.cpu(), eps, wanted, None if picked is None else picked.cpu(),
                                   branch.cpu() if use_branch else None)
            close(found, wanted, dtype)
            assert torch.equal(values, before)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(1, 64), (4, 97), (3, 2050), (8, 4096), (70, 1024), (2, 5120), (2, 9000)])
def test_add_rms_norm(dtype, rows, width):
    branch = randn(rows, width, dtype=dtype, seed=5)
    residual = randn(rows, width, dtype=dtype, seed=6, scale=2.0)
    weight = (1 + 0.1 * torch.randn(width, generator=torch.Generator().manual_seed(7))).to(DEVICE)
    wanted_residual, wanted = residual.cpu().clone(), torch.empty(rows, width, dtype=dtype)
    plain_kernels.add_rms_norm(branch.cpu(), wanted_residual, weight.cpu(), 1e-6, wanted)
    found = torch.empty_like(residual)
    kernels.add_rms_norm(branch, residual, weight, 1e-6, found)
    assert torch.equal(residual.cpu(), wanted_residual)   # one rounded sum, the same on both sides
    close(found, wanted, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(1, 1), (3, 225), (70, 1000), (8, 12288), (33, 72)])
def test_silu_mul(dtype, rows, width):
    stacked = randn(rows, 2 * width, dtype=dtype, seed=8, scale=4.0)
    found = torch.empty(rows, width, dtype=dtype, device=DEVICE)
    wanted = torch.empty(rows, width, dtype=dtype)
    kernels.silu_mul(stacked, found)
    plain_kernels.silu_mul(stacked.cpu(), wanted)
    close(found, wanted, dtype)


@pytest.mark.parametrize("dtype,out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (3, 70, 33), (65, 130, 100), (128, 64, 256), (9, 500, 96)])
def test_gemm_simt(dtype, out_dtype, m, n, k):
    values = randn(m, k, dtype=dtype, seed=9)
    weight = randn(n, k, dtype=dtype, seed=10)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(11)).to(DEVICE)
    for use_bias in (None, bias):
        found = torch.empty(m, n, dtype=out_dtype, device=DEVICE)
        wanted = torch.empty(m, n, dtype=out_dtype)
        kernels.gemm_simt(values, weight, use_bias, found)
        plain_kernels.linear(values.cpu(), weight.cpu(), None if use_bias is None else use_bias.cpu(), wanted)
        close(found, wanted, out_dtype)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k", [(1, 16, 8), (8, 100, 72), (3, 17, 4096), (9, 33, 520), (16, 256, 128), (17, 40, 200), (32, 1000, 64)])
def test_gemm_skinny(out_dtype, m, n, k):
    values = randn(m, k + 8, dtype=torch.bfloat16, seed=15)[:, :k]     # rows wider than K
    weight = randn(n, k, dtype=torch.bfloat16, seed=16)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(17)).to(DEVICE)
    for use_bias in (None, bias):
        found = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEVICE)
        wanted = torch.empty(m, n, dtype=out_dtype)
        kernels.gemm_skinny(values, weight, use_bias, found)
        plain_kernels.linear(values.cpu(), weight.cpu(), None if use_bias is None else use_bias.cpu(), wanted)
        close(found, wanted, out_dtype)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k,box", [(1, 8, 8, 0), (16, 128, 64, 0), (33, 130, 72, 0), (128, 128, 128, 0), (200, 300, 200, 0),
                                       (257, 129, 520, 0), (700, 260, 1032, 0), (40, 500, 96, 16), (100, 257, 136, 32),
                                       (300, 100, 64, 128), (64, 1000, 224, 256), (500, 260, 136, 192), (193, 129, 72, 192), (512, 6144, 256, 0), (1024, 700, 64, 0)])
def test_gemm_tc(out_dtype, m, n, k, box):
    """The tcgen05 product at ragged sizes (zero-filled tails in every direction), every token tile, strided views."""
    values = randn(m, k + 8, dtype=torch.bfloat16, seed=18)[:, :k]
    weight = randn(n + 3, k, dtype=torch.bfloat16, seed=19)[:n]
    bias = torch.randn(n, generator=torch.Generator().manual_seed(20)).to(DEVICE)
    for use_bias in (None, bias):
        found = torch.full((m, n + 5), float("nan"), dtype=out_dtype, device=DEVICE)[:, :n]
        wanted = torch.empty(m, n, dtype=out_dtype)
        plain_kernels.linear(values.cpu(), weight.cpu(), None if use_bias is None else use_bias.cpu(), wanted)
        for pair in ((0, 1) if (box == 256 or (box == 0 and m > 128)) else (-1,)):   # one SM per tile, and pairs of SMs on 256 x 256 tiles
            found.fill_(float("nan"))
            kernels.gemm_tc(values, weight, use_bias, found, box, pair=pair)
            close(found, wanted, out_dtype)
    assert kernels.gemm_tc_status() == 0


@pytest.mark.parametrize("m,n,k", [(1, 16, 8), (8, 48, 72), (20, 240, 200), (32, 1000 // 16 * 16, 64), (33, 64, 136), (200, 400, 96), (300, 16, 520)])
def test_gated_products(m, n, k):
    """silu(gate) * up as the epilogue of the skinny and of the tcgen05 product, on interleaved gate/up rows."""
    values = randn(m, k, dtype=torch.bfloat16, seed=21)
    weight = randn(n, k, dtype=torch.bfloat16, seed=22)
    wanted = torch.empty(m, n // 2, dtype=torch.bfloat16)
    plain_kernels.linear_gated(values.cpu(), weight.cpu(), wanted)
    found = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device=DEVICE)
    kernels.linear_gated(values, weight, found)
    close(found, wanted, torch.bfloat16)
    for pair in (0, -1):
        found.fill_(float("nan"))
        kernels.gemm_tc(values, weight, None, found, gated=True, pair=pair)
        close(found, wanted, torch.bfloat16)
    assert kernels.gemm_tc_status() == 0


@pytest.mark.parametrize("m,n,k,splits", [(40, 130, 520, 2), (64, 260, 1032, 3), (33, 128, 4096, 8), (128, 500, 584, 5), (20, 1000, 264, 4),
                                          (200, 140, 520, 3), (64, 4096, 2048, 0), (48, 512, 4096, 0)])
def test_gemm_tc_cut_along_k(m, n, k, splits):
    """K ranges of a tile meet in the workspace; the last warp to arrive adds them in a fixed order.  Ragged sizes, every
    epilogue, a second launch on the tickets that the first one left, and the same bits whoever finishes last."""
    values = randn(m, k, dtype=torch.bfloat16, seed=23)
    weight = randn(n, k, dtype=torch.bfloat16, seed=24)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(25)).to(DEVICE)
    for out_dtype in (torch.bfloat16, torch.float32):
        wanted = torch.empty(m, n, dtype=out_dtype)
        plain_kernels.linear(values.cpu(), weight.cpu(), bias.cpu(), wanted)
        first = None
        for attempt in range(4):   # the ranges meet in a cluster's shared memory, or in the workspace: the same sums in the same order
            found = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEVICE)
            kernels.gemm_tc(values, weight, bias, found, splits=splits, cluster=attempt % 2 == 0)
            close(found, wanted, out_dtype)
            first = found if first is None else first
            assert torch.equal(found, first)
    if n % 16 == 0:
        wanted = torch.empty(m, n // 2, dtype=torch.bfloat16)
        plain_kernels.linear_gated(values.cpu(), weight.cpu(), wanted)
        found = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device=DEVICE)
        for cluster in (True, False):
            found.fill_(float("nan"))
            kernels.gemm_tc(values, weight, None, found, gated=True, splits=splits, cluster=cluster)
            close(found, wanted, torch.bfloat16)
    assert kernels.gemm_tc_status() == 0
    with pytest.raises(Exception):
        kernels.gemm_tc(values, weight, bias, torch.empty(m, n, dtype=torch.bfloat16, device=DEVICE), splits=k // 64 + 2)   # more ranges than K blocks


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_dispatch_matches_plain(dtype):
    """Whatever kernel `linear` picks for a shape, the product is the same: ragged and aligned shapes, views of a stack."""
    for m, n, k in [(1, 64, 64), (8, 6144 // 8, 512), (17, 257, 136), (64, 96, 224), (200, 128, 128), (5, 500, 96)]:
        values = randn(m, k, dtype=dtype, seed=12)
        stack = randn(n + 16, k, dtype=dtype, seed=13)
        weight = stack[:n]
        bias = torch.randn(n, generator=torch.Generator().manual_seed(14)).to(DEVICE)
        for out_dtype in {dtype, torch.float32}:
            found = torch.empty(m, n, dtype=out_dtype, device=DEVICE)
            wanted = torch.empty(m, n, dtype=out_dtype)
            kernels.linear(values, weight, bias, found)
            plain_kernels.linear(values.cpu(), weight.cpu(), bias.cpu(), wanted)
            close(found, wanted, out_dtype)


def paged_setup(lengths, new_counts, n_kv_heads, head_dim, dtype, seed, pages=40):
    """Random cache pages, page rows that scatter each sequence over the pool, and the step's metadata."""
    rng = np.random.default_rng(seed)
    keys = randn(pages, n_kv_heads, 64, head_dim, dtype=dtype, seed=seed + 1)
    values = randn(pages, n_kv_heads, 64, head_dim, dtype=dtype, seed=seed + 2)
    order = rng.permutation(pages)
    stride = max((length + 63) // 64 for length in lengths)
    rows = np.zeros((len(lengths), stride), dtype=np.int32)
    cursor = 0
    for index, length in enumerate(lengths):
        count = (length + 63) // 64
        rows[index, :count] = order[cursor : cursor + count]
        cursor += count
    positions, token_seq = [], []
    for index, (length, new) in enumerate(zip(lengths, new_counts)):
        positions += list(range(length - new, length))
        token_seq += [index] * new
    to_device = lambda array: torch.tensor(np.asarray(array), dtype=torch.int32, device=DEVICE)
    return keys, values, to_device(rows), to_device(positions), to_device(token_seq)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,rotary_dim,with_norm", [
    (4, 2, 16, 16, True), (6, 3, 48, 48, True), (8, 1, 32, 16, True), (3, 3, 128, 128, False), (2, 1, 256, 0, True),
    (8, 2, 64, 64, True), (5, 1, 128, 128, True), (2, 2, 256, 256, True), (4, 2, 128, 64, True)])
def test_attention_prepare(dtype, n_heads, n_kv_heads, head_dim, rotary_dim, with_norm):
    lengths, new_counts = [70, 5, 129], [70, 1, 3]
    keys, values, rows, positions, token_seq = paged_setup(lengths, new_counts, n_kv_heads, head_dim, dtype, seed=20)
    tokens = positions.shape[0]
    width = (n_heads + 2 * n_kv_heads) * head_dim
    projected = randn(tokens, width + 8, dtype=dtype, seed=21)[:, :width]   # a view with a wider row stride
    generator = torch.Generator().manual_seed(22)
    q_weight = (1 + 0.1 * torch.randn(head_dim, generator=generator)).to(DEVICE) if with_norm else None
    k_weight = (1 + 0.1 * torch.randn(head_dim, generator=generator)).to(DEVICE) if with_norm else None
    angles = torch.rand(200, max(rotary_dim // 2, 1), generator=generator) * 6.0
    cos, sin = (torch.cos(angles).to(DEVICE), torch.sin(angles).to(DEVICE)) if rotary_dim else (None, None)
    for write in (True, False):
        found_q = torch.empty(tokens, n_heads * head_dim, dtype=dtype, device=DEVICE)
        found_k, found_v = keys.clone(), values.clone()
        kernels.attention_prepare(projected, found_q, found_k, found_v, write, q_weight, k_weight, 1e-5, cos, sin, rotary_dim,
                                  positions, token_seq, rows, n_heads, n_kv_heads, head_dim)
        cpu = lambda t: None if t is None else t.cpu()
        wanted_q = torch.empty(tokens, n_heads * head_dim, dtype=dtype)
        wanted_k, wanted_v = keys.cpu().clone(), values.cpu().clone()
        plain_kernels.attention_prepare(projected.cpu(), wanted_q, wanted_k, wanted_v, write, cpu(q_weight), cpu(k_weight), 1e-5,
                                        cpu(cos), cpu(sin), rotary_dim, positions.cpu(), token_seq.cpu(), rows.cpu(), n_heads,
                                        n_kv_heads, head_dim)
        close(found_q, wanted_q, dtype)
        close(found_k, wanted_k, dtype)
        assert torch.equal(found_v.cpu(), wanted_v)
        untouched = (wanted_k == keys.cpu())
        assert torch.equal(found_k.cpu()[untouched], keys.cpu()[untouched])   # nothing else in the pool is written


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,window", [
    (4, 2, 16, 0), (6, 3, 48, 0), (8, 1, 32, 0), (5, 5, 128, 0), (2, 1, 256, 0), (4, 2, 64, 37)])
def test_attention_over_pages(dtype, n_heads, n_kv_heads, head_dim, window):
    """Prompts, single tokens and continued runs in one launch, against the plain statement."""
    lengths, new_counts = [70, 200, 129, 1, 64], [70, 1, 3, 1, 1]
    keys, values, rows, positions, token_seq = paged_setup(lengths, new_counts, n_kv_heads, head_dim, dtype, seed=30)
    tokens = positions.shape[0]
    queries = randn(tokens, n_heads * head_dim, dtype=dtype, seed=31)
    found = torch.empty_like(queries)
    wanted = torch.empty(tokens, n_heads * head_dim, dtype=dtype)
    scale = head_dim ** -0.5

    class Step:
        pass

    step = Step()
    step.positions, step.token_seq, step.n_tokens, step.n_seqs = positions, token_seq, tokens, len(lengths)
    step.max_new, step.max_len, step.all_single, step.decode_splits = max(new_counts), max(lengths), False, 0
    step.cu_seqlens = torch.tensor(np.concatenate([[0], np.cumsum(new_counts)]), dtype=torch.int32, device=DEVICE)
    step.seq_start = torch.tensor([l - n for l, n in zip(lengths, new_counts)], dtype=torch.int32, device=DEVICE)
    step.seq_len = torch.tensor(lengths, dtype=torch.int32, device=DEVICE)
    kernels.attention(queries, keys, values, found, step, rows, n_heads, n_kv_heads, head_dim, scale, window)
    plain_kernels.attention_generic(queries.cpu(), keys.cpu(), values.cpu(), wanted, positions.cpu(), token_seq.cpu(), rows.cpu(),
                                    n_heads, n_kv_heads, head_dim, scale, window)
    close(found, wanted, dtype)


@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,window", [
    (4, 4, 16, 0), (6, 2, 48, 0), (8, 2, 128, 0), (10, 2, 64, 0), (3, 1, 256, 0), (2, 1, 80, 0), (8, 2, 128, 50), (4, 2, 32, 16)])
def test_prefill_attention_kernel(n_heads, n_kv_heads, head_dim, window):
    """The tensor-core prefill kernel on whole prompts, continued runs, ragged tiles and a window's edge."""
    dtype = torch.bfloat16
    lengths, new_counts = [70, 200, 129, 1, 64, 333], [70, 17, 129, 1, 33, 100]
    keys, values, rows, positions, token_seq = paged_setup(lengths, new_counts, n_kv_heads, head_dim, dtype, seed=70, pages=48)
    tokens = positions.shape[0]
    queries = randn(tokens, n_heads * head_dim, dtype=dtype, seed=71)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(new_counts)]), dtype=torch.int32, device=DEVICE)
    starts = torch.tensor([l - n for l, n in zip(lengths, new_counts)], dtype=torch.int32, device=DEVICE)
    # Poison what lies beyond each sequence's length: nothing there may be read into a result.
    for index, length in enumerate(lengths):
        for place in range(length, ((length + 63) // 64) * 64):
            keys[int(rows[index, place // 64]), :, place % 64] = float("nan")
            values[int(rows[index, place // 64]), :, place % 64] = float("nan")
    found = torch.full_like(queries, float("nan"))
    wanted = torch.empty(tokens, n_heads * head_dim, dtype=dtype)
    kernels.attention_prefill(queries, keys, values, found, cu, starts, rows, n_heads, n_kv_heads, head_dim, head_dim ** -0.5, window)
    plain_kernels.attention_generic(queries.cpu(), keys.cpu(), values.cpu(), wanted, positions.cpu(), token_seq.cpu(), rows.cpu(),
                                    n_heads, n_kv_heads, head_dim, head_dim ** -0.5, window)
    close(found, wanted, dtype)


@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,window", [(8, 2, 128, 0), (4, 4, 64, 0), (6, 1, 128, 0), (4, 2, 128, 50), (2, 1, 64, 130)])
def test_prefill_attention_tensor_memory_kernel(n_heads, n_kv_heads, head_dim, window):
    """The tcgen05 prefill kernel: whole prompts, continued runs, ragged 128-row tiles, several pages, a window's edge,
    a far key that must dominate; poisoned rows beyond each length must not be read into a result."""
    dtype = torch.bfloat16
    lengths, new_counts = [70, 200, 129, 1, 64, 700, 128], [70, 17, 129, 1, 33, 300, 128]
    keys, values, rows, positions, token_seq = paged_setup(lengths, new_counts, n_kv_heads, head_dim, dtype, seed=90, pages=64)
    tokens = positions.shape[0]
    queries = randn(tokens, n_heads * head_dim, dtype=dtype, seed=91)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(new_counts)]), dtype=torch.int32, device=DEVICE)
    starts = torch.tensor([l - n for l, n in zip(lengths, new_counts)], dtype=torch.int32, device=DEVICE)
    if window == 0:   # the last token of the longest request finds key 5 among 700
        last = int(cu[6]) - 1
        query = queries[last].view(n_heads, head_dim)[0].float()
        keys[int(rows[5, 0]), 0, 5] = (query * 60.0 / query.norm()).to(dtype)
    for index, length in enumerate(lengths):
        for place in range(length, ((length + 63) // 64) * 64):
            keys[int(rows[index, place // 64]), :, place % 64] = float("nan")
            values[int(rows[index, place // 64]), :, place % 64] = float("nan")
    found = torch.full_like(queries, float("nan"))
    wanted = torch.empty(tokens, n_heads * head_dim, dtype=dtype)
    kernels.attention_prefill_tc(queries, keys, values, found, cu, starts, rows, n_heads, n_kv_heads, head_dim, head_dim ** -0.5, window)
    plain_kernels.attention_generic(queries.cpu(), keys.cpu(), values.cpu(), wanted, positions.cpu(), token_seq.cpu(), rows.cpu(),
                                    n_heads, n_kv_heads, head_dim, head_dim ** -0.5, window)
    close(found, wanted, dtype)
    assert kernels.attention_prefill_tc_status(head_dim) == 0
    if window == 0:
        got = found[int(cu[6]) - 1].view(n_heads, head_dim)[0].float()
        assert torch.allclose(got, values[int(rows[5, 0]), 0, 5].float(), atol=0.05, rtol=0.05)


def test_prefill_attention_shares_more_tiles_than_blocks_out_and_leaves_its_counter_at_zero():
    """The tcgen05 prefill kernel's blocks stay and take tiles off a counter: 40 prompts of unequal lengths and 4 heads are
    more tiles than the device holds blocks, every one must be done exactly once (a tile done twice shows nowhere, so
    the output starts as NaN and a tile left out stays NaN), and three launches in a row on the same counter agree."""
    dtype, n_heads, n_kv_heads, head_dim = torch.bfloat16, 4, 2, 128
    generator = np.random.default_rng(17)
    lengths = [int(v) for v in generator.integers(1, 400, size=40)]
    new_counts = [length if index % 3 else max(1, length // 2) for index, length in enumerate(lengths)]   # a third of them continue
    keys, values, rows, positions, token_seq = paged_setup(lengths, new_counts, n_kv_heads, head_dim, dtype, seed=92, pages=sum((l + 63) // 64 for l in lengths) + 3)
    tokens = positions.shape[0]
    assert (tokens // 128 + len(lengths)) * n_heads > 2 * kernels.sm_count(DEVICE)
    queries = randn(tokens, n_heads * head_dim, dtype=dtype, seed=93)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(new_counts)]), dtype=torch.int32, device=DEVICE)
    starts = torch.tensor([l - n for l, n in zip(lengths, new_counts)], dtype=torch.int32, device=DEVICE)
    wanted = torch.empty(tokens, n_heads * head_dim, dtype=dtype)
    plain_kernels.attention_generic(queries.cpu(), keys.cpu(), values.cpu(), wanted, positions.cpu(), token_seq.cpu(), rows.cpu(),
                                    n_heads, n_kv_heads, head_dim, head_dim ** -0.5, 0)
    results = []
    for _ in range(3):
        found = torch.full_like(queries, float("nan"))
        kernels.attention_prefill_tc(queries, keys, values, found, cu, starts, rows, n_heads, n_kv_heads, head_dim, head_dim ** -0.5, 0)
        assert kernels.attention_prefill_tc_status(head_dim) == 0
        close(found, wanted, dtype)
        results.append(found)
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])
    for schedule in kernels._prefill_schedule.values():
        assert int(schedule.abs().sum()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim", [(4, 2, 16), (8, 2, 128), (6, 1, 80)])
def test_decode_attention_finds_a_far_key(dtype, n_heads, n_kv_heads, head_dim):
    """One token per sequence over long contexts; one far key is scaled so that its value must dominate."""
    lengths = [1500, 63, 1025, 700]
    keys, values, rows, positions, token_seq = paged_setup(lengths, [1] * 4, n_kv_heads, head_dim, dtype, seed=40, pages=64)
    queries = randn(4, n_heads * head_dim, dtype=dtype, seed=41)
    far = [3, 0, 1000, 64]
    for index, place in enumerate(far):
        page = int(rows[index, place // 64])
        for head in range(n_kv_heads):
            query = queries[index].view(n_heads, head_dim)[head * (n_heads // n_kv_heads)].float()
            keys[page, head, place % 64] = (query * 40.0 / query.norm()).to(dtype)
    found = torch.empty_like(queries)
    wanted = torch.empty(4, n_heads * head_dim, dtype=dtype)

    class Step:
        pass

    step = Step()
    step.positions, step.token_seq, step.n_tokens, step.n_seqs = positions, token_seq, 4, 4
    step.max_new, step.max_len, step.all_single, step.decode_splits = 1, max(lengths), True, 0
    step.cu_seqlens = torch.arange(5, dtype=torch.int32, device=DEVICE)
    step.seq_start = torch.tensor([l - 1 for l in lengths], dtype=torch.int32, device=DEVICE)
    step.seq_len = torch.tensor(lengths, dtype=torch.int32, device=DEVICE)
    kernels.attention(queries, keys, values, found, step, rows, n_heads, n_kv_heads, head_dim, head_dim ** -0.5, 0)
    plain_kernels.attention_generic(queries.cpu(), keys.cpu(), values.cpu(), wanted, positions.cpu(), token_seq.cpu(), rows.cpu(),
                                    n_heads, n_kv_heads, head_dim, head_dim ** -0.5, 0)
    close(found, wanted, dtype)
    for index, place in enumerate(far):   # the first head of each group reproduces the far value
        page = int(rows[index, place // 64])
        got = found[index].view(n_heads, head_dim)[0].float()
        assert torch.allclose(got, values[page, 0, place % 64].float(), atol=0.05, rtol=0.05)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,window", [
    (3, 3, 32, 0), (10, 2, 64, 0), (16, 1, 16, 0), (12, 4, 96, 0), (8, 2, 256, 0), (4, 1, 128, 100)])
def test_decode_attention_splits_and_groups(dtype, n_heads, n_kv_heads, head_dim, window):
    """Every number of splits gives the same context: groups of 1, 3, 4, 5 and 16 heads, splits that are empty
    for short sequences, a window."""
    lengths = [1, 33, 300, 129, 64]
    keys, values, rows, positions, token_seq = paged_setup(lengths, [1] * 5, n_kv_heads, head_dim, dtype, seed=60, pages=24)
    queries = randn(5, n_heads * head_dim, dtype=dtype, seed=61)
    seq_len = torch.tensor(lengths, dtype=torch.int32, device=DEVICE)
    wanted = torch.empty(5, n_heads * head_dim, dtype=dtype)
    plain_kernels.attention_generic(queries.cpu(), keys.cpu(), values.cpu(), wanted, positions.cpu(), token_seq.cpu(), rows.cpu(),
                                    n_heads, n_kv_heads, head_dim, head_dim ** -0.5, window)
    for splits in (1, 2, 5, 8, 13, 16, 24):
        for cluster_merge in (True, False):   # up to 16 splits meet in a cluster's shared memory, or like more of them in global memory
            found = torch.full_like(queries, float("nan"))
            kernels.attention_decode(queries, keys, values, found, seq_len, rows, n_heads, n_kv_heads, head_dim, head_dim ** -0.5, window, splits,
                                     cluster_merge=cluster_merge)
            close(found, wanted, dtype)


@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,rotary_dim,with_norm,window", [
    (8, 2, 128, 128, True, 0), (4, 4, 16, 16, True, 0), (6, 3, 48, 16, False, 0), (16, 1, 64, 64, True, 0), (4, 1, 32, 32, True, 20)])
def test_fused_decode_attention(n_heads, n_kv_heads, head_dim, rotary_dim, with_norm, window):
    """Norm, rotation, cache write and split attention in one kernel against the plain prepare followed by plain attention."""
    dtype = torch.bfloat16
    lengths = [1, 64, 65, 300, 130]
    keys, values, rows, positions, token_seq = paged_setup(lengths, [1] * 5, n_kv_heads, head_dim, dtype, seed=80, pages=24)
    width = (n_heads + 2 * n_kv_heads) * head_dim
    projected = randn(5, width, dtype=dtype, seed=81)
    generator = torch.Generator().manual_seed(82)
    q_weight = (1 + 0.1 * torch.randn(head_dim, generator=generator)).to(DEVICE) if with_norm else None
    k_weight = (1 + 0.1 * torch.randn(head_dim, generator=generator)).to(DEVICE) if with_norm else None
    angles = torch.rand(400, rotary_dim // 2, generator=generator) * 6.0
    cos, sin = torch.cos(angles).to(DEVICE), torch.sin(angles).to(DEVICE)
    seq_len = torch.tensor(lengths, dtype=torch.int32, device=DEVICE)
    cpu = lambda t: None if t is None else t.cpu()
    for write in (True, False):
        wanted_k, wanted_v = keys.cpu().clone(), values.cpu().clone()
        wanted_q = torch.empty(5, n_heads * head_dim, dtype=dtype)
        plain_kernels.attention_prepare(projected.cpu(), wanted_q, wanted_k, wanted_v, write, cpu(q_weight), cpu(k_weight), 1e-6, cpu(cos),
                                        cpu(sin), rotary_dim, positions.cpu(), token_seq.cpu(), rows.cpu(), n_heads, n_kv_heads, head_dim)
        wanted = torch.empty(5, n_heads * head_dim, dtype=dtype)
        plain_kernels.attention_generic(wanted_q, wanted_k, wanted_v, wanted, positions.cpu(), token_seq.cpu(), rows.cpu(), n_heads,
                                        n_kv_heads, head_dim, head_dim ** -0.5, window)
        for splits in (1, 3, 8):
            found_k, found_v = keys.clone(), values.clone()
            found = torch.full((5, n_heads * head_dim), float("nan"), dtype=dtype, device=DEVICE)
            kernels.attention_decode(None, found_k, found_v, found, seq_len, rows, n_heads, n_kv_heads, head_dim, head_dim ** -0.5, window,
                                     splits, prepare=(projected, q_weight, k_weight, 1e-6, cos, sin, rotary_dim, write))
            close(found, wanted, dtype)
            close(found_k, wanted_k, dtype)
            assert torch.equal(found_v.cpu(), wanted_v)
            kernels.attention_decode(None, found_k, found_v, found, seq_len, rows, n_heads, n_kv_heads, head_dim, head_dim ** -0.5, window,
                                     splits, prepare=(projected, q_weight, k_weight, 1e-6, cos, sin, rotary_dim, write))
            close(found, wanted, dtype)     # a second launch finds the tickets at zero again


def adversarial_rows():
    nan, inf = float("nan"), float("inf")
    rows = [
        [nan, nan, nan], [nan, -inf, nan], [1.0, 2.0, 2.0, 1.0], [2.0, 1.0, 2.0], [-0.0, 0.0, -0.0], [0.0, -0.0],
        [inf, 3.0, inf], [-inf, -inf], [nan, 5.0, nan, 5.0, nan], [1e-45, 0.0, -1e-45], [-1.0, -2.0, -1.0],
    ]
    return rows


def test_argmax_semantics():
    """The reference's cases: NaN never wins, +-inf, signed zeros, subnormals, ties go to the highest id
    (crates/engine/src/generation/greedy/tests.rs:18-48)."""
    for row in adversarial_rows():
        logits = torch.tensor([row], dtype=torch.float32, device=DEVICE)
        tokens = torch.full((1,), -7, dtype=torch.int32, device=DEVICE)
        valid = torch.full((1,), -7, dtype=torch.int32, device=DEVICE)
        kernels.argmax(logits, tokens, valid)
        token, ok = plain_kernels.argmax_row(np.asarray(row, dtype=np.float32))
        assert int(valid[0]) == ok, row
        if ok:
            assert int(tokens[0]) == token, row


@pytest.mark.parametrize("vocab", [1, 31, 32, 33, 255, 256, 257, 2047, 2048, 2049, 151936])
def test_argmax_random_bit_patterns(vocab):
    rng = np.random.default_rng(vocab)
    bits = rng.integers(0, 2 ** 32, size=(5, vocab), dtype=np.uint64).astype(np.uint32)
    bits[1, :] = bits[1, 0]                      # all equal: the last index wins
    bits[2, :] = 0x7FC00000                      # all NaN
    if vocab > 2:
        bits[3, vocab // 2] = 0x7F800000         # one +inf
        bits[3, -1] = 0x7F800000                 # ... and a later one
    values = bits.view(np.float32)
    logits = torch.from_numpy(values.copy()).to(DEVICE)
    tokens = torch.empty(5, dtype=torch.int32, device=DEVICE)
    valid = torch.empty(5, dtype=torch.int32, device=DEVICE)
    kernels.argmax(logits, tokens, valid)
    for row in range(5):
        token, ok = plain_kernels.argmax_row(values[row])
        assert int(valid[row]) == ok
        if ok:
            assert int(tokens[row]) == token


def test_gumbel_sampling_matches_plain_and_distribution():
    vocab, rows = 700, 6
    logits = torch.randn(rows, vocab, generator=torch.Generator().manual_seed(50)) * 2.0
    logits[2, 5] = float("nan")
    device_logits = logits.to(DEVICE)
    requests = torch.tensor([0, 1, 2, 3, 4, 4], dtype=torch.int32, device=DEVICE)
    indices = torch.tensor([0, 0, 9, 1, 7, 8], dtype=torch.int32, device=DEVICE)
    tokens = torch.empty(rows, dtype=torch.int32, device=DEVICE)
    valid = torch.empty(rows, dtype=torch.int32, device=DEVICE)
    kernels.sample_gumbel(device_logits, tokens, valid, 1.0 / 0.8, 1234567890123, requests, indices)
    for row in range(rows):
        scores = plain_kernels.gumbel_scores(logits[row].numpy(), 1.0 / 0.8, 1234567890123, int(requests[row]), int(indices[row]))
        best = np.nanmax(scores)
        assert int(valid[row]) == 1
        assert scores[int(tokens[row])] >= best - 1e-4 * max(1.0, abs(best))   # log differs in the last bits only
    # The same request and token index give the same token whatever else is in the batch.
    alone = torch.empty(1, dtype=torch.int32, device=DEVICE)
    kernels.sample_gumbel(device_logits[4:5].contiguous(), alone, valid[:1].clone(), 1.0 / 0.8, 1234567890123, requests[4:5], indices[4:5])
    assert int(alone[0]) == int(tokens[4])
    # Frequencies follow softmax(logits / T).
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0, float("-inf")]], device=DEVICE).repeat(4000, 1).contiguous()
    draws = torch.empty(4000, dtype=torch.int32, device=DEVICE)
    kernels.sample_gumbel(small, draws, torch.empty(4000, dtype=torch.int32, device=DEVICE), 1.0 / 0.5, 7,
                          torch.arange(4000, dtype=torch.int32, device=DEVICE), torch.zeros(4000, dtype=torch.int32, device=DEVICE))
    counts = torch.bincount(draws.long().cpu(), minlength=5).double() / 4000
    expected = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0, float("-inf")]).double() / 0.5, dim=0)
    assert float((counts - expected).abs().max()) < 0.03


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("count,scale,shift", [(1, 0.02, 0.0), (5, 0.02, 0.0), (4099, 0.1, 1.0), (3_000_001, 0.02, 0.0)])
def test_random_weights_are_the_same_bits_on_the_device_and_on_the_host(dtype, count, scale, shift):
    """The device's draw of a tensor against the host's (numpy): every bit equal, in float32 and after the rounding to
    bfloat16, for counts that are no multiple of four and for both kinds of tensor (N(0, s) and 1 + N(0, s))."""
    from tau_rs_b200.weights import TensorSpec, random_tensor

    spec = TensorSpec((count,), role="vector" if shift else "matrix", init="ones" if shift else "normal", std=scale)
    host = random_tensor("model.layers.3.some.weight", spec, seed=11, norm_jitter=scale, device="cpu", dtype=dtype)
    device = random_tensor("model.layers.3.some.weight", spec, seed=11, norm_jitter=scale, device=DEVICE, dtype=dtype)
    assert device.dtype == dtype and device.is_cuda
    assert torch.equal(device.cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                       host.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
    other = random_tensor("model.layers.4.some.weight", spec, seed=11, norm_jitter=scale, device=DEVICE, dtype=dtype)
    assert count < 5 or not torch.equal(other, device)


def test_a_model_drawn_on_the_device_equals_the_folder_written_on_the_host(tmp_path):
    """`random_model` (no file) against `write_random_model` + `load_model` for the same configuration and seed."""
    import tiny_configs
    from tau_rs_b200 import load_model
    from tau_rs_b200.api import random_model

    for which, dtype in (("B", "float32"), ("C", "bfloat16")):
        folder = tiny_configs.write_tiny(str(tmp_path), which, dtype)
        loaded = load_model(folder, dtype, "gpu")
        drawn = random_model(dict(tiny_configs.CONFIGS[which], torch_dtype=dtype), seed=tiny_configs.SEEDS[which], dtype=dtype, norm_jitter=0.1)
        assert torch.equal(loaded.embedding, drawn.embedding) and torch.equal(loaded.head, drawn.head)
        for a, b in zip(loaded.blocks, drawn.blocks):
            assert torch.equal(a.mixer.qkv.weight, b.mixer.qkv.weight) and torch.equal(a.mixer.q_norm.weight, b.mixer.q_norm.weight)
            assert torch.equal(a.feed_forward.gate_up.weight, b.feed_forward.gate_up.weight)
            assert torch.equal(a.feed_forward.down.weight, b.feed_forward.down.weight)
            if a.mixer.qkv.bias is not None:
                assert torch.equal(a.mixer.qkv.bias, b.mixer.qkv.bias)


def test_argmax_calls_in_a_row_share_their_scratch():
    """Calls of changing sizes one after another on one stream (the tickets at the start of the scratch go back to zero
    after every call), rows of NaN between valid ones (no token of an earlier call survives: crates/engine/src/
    generation/greedy/tests.rs:125-156), and more rows than one launch has tickets for."""
    generator = torch.Generator().manual_seed(60)
    for rows, vocab in ((3, 5000), (64, 151936), (1, 7), (9000, 40), (3, 5000), (2, 4099)):
        logits = torch.randn(rows, vocab, generator=generator)
        logits[rows // 2, :] = float("nan")
        logits[0, -1] = logits[0].max()
        device_logits = logits.to(DEVICE)
        tokens = torch.full((rows,), -7, dtype=torch.int32, device=DEVICE)
        valid = torch.full((rows,), -7, dtype=torch.int32, device=DEVICE)
        for _ in range(2):
            kernels.argmax(device_logits, tokens, valid)
        wanted = torch.where(torch.isnan(logits), torch.full_like(logits, -float("inf")), logits)
        best = wanted.max(dim=1, keepdim=True).values
        last_best = (vocab - 1) - torch.flip(wanted == best, dims=[1]).int().argmax(dim=1)
        is_valid = ~torch.isnan(logits).all(dim=1)
        assert torch.equal(valid.cpu().bool(), is_valid)
        assert torch.equal(tokens.cpu()[is_valid].long(), last_best[is_valid])
        assert int(tokens[rows // 2]) == 0 and int(valid[rows // 2]) == 0


@pytest.mark.parametrize("head_dim,length", [(128, 6000), (64, 4000)])
def test_prefill_attention_counts_every_key_tile_of_a_long_context(head_dim, length):
    """Thousands of positions with inputs made so that a lost key tile shows in every row: all queries are zero, so a row
    attends evenly to every key it may see, and the value of key k is 1 in column k // 64 and 0 elsewhere; row p must then
    hold `visible keys of tile c / (p + 1)` in column c, exactly up to the output's rounding.  Whole, and as a second run
    behind 3,000 cached positions (one wrong row among thousands was how a race in the hand-over of value tiles once showed)."""
    n_heads, n_kv_heads = 2, 1
    assert length // 64 < head_dim
    n_pages = (length + 63) // 64
    generator = torch.Generator().manual_seed(7)
    order = torch.randperm(n_pages + 5, generator=generator)[:n_pages].to(torch.int32)
    keys = torch.randn(n_pages + 5, n_kv_heads, 64, head_dim, generator=generator).to(torch.bfloat16).to(DEVICE)
    values = torch.zeros(n_pages + 5, n_kv_heads, 64, head_dim, dtype=torch.bfloat16, device=DEVICE)
    for tile in range(n_pages):
        values[int(order[tile]), 0, :, tile] = 1.0
        if tile == n_pages - 1 and length % 64:
            values[int(order[tile]), 0, length % 64:] = float("nan")      # beyond the sequence: never read into a result
    rows = order.view(1, n_pages).to(DEVICE).contiguous()
    position = torch.arange(length, dtype=torch.float32)
    wanted = torch.zeros(length, head_dim)
    for tile in range(n_pages):
        wanted[:, tile] = (position + 1 - 64 * tile).clamp(0, 64) / (position + 1)
    for start in (0, 3000):
        new = length - start
        queries = torch.zeros(new, n_heads * head_dim, dtype=torch.bfloat16, device=DEVICE)
        found = torch.full_like(queries, float("nan"))
        cu = torch.tensor([0, new], dtype=torch.int32, device=DEVICE)
        starts = torch.tensor([start], dtype=torch.int32, device=DEVICE)
        kernels.attention_prefill_tc(queries, keys, values, found, cu, starts, rows, n_heads, n_kv_heads, head_dim, head_dim ** -0.5, 0)
        assert kernels.attention_prefill_tc_status(head_dim) == 0
        for head in range(n_heads):
            got = found.view(new, n_heads, head_dim)[:, head].float().cpu()
            error = (got - wanted[start:]).abs()
            worst = int(error.max(dim=1).values.argmax())
            assert float(error.max()) <= 2 ** -8 * float(wanted[start:].max()), (start, head, start + worst, float(error.max()))
