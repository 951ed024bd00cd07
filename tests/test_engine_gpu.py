"""The engine on the GPU against the plain whole-sequence implementation, in every way of cutting the work."""
import pytest
import torch

import plain_model
import tiny_configs
from helpers import (engine_for, plain_logits, random_prompts, relative_error, run_batched, run_tail_stepwise, run_whole)
from tau_rs_b200 import StepEntry, generate

pytestmark = pytest.mark.gpu
# Largest difference relative to the largest logit.  32-bit: rounding of sums only.  bfloat16: the plain
# implementation rounds where the engine stores, so what is left are roundings that fall the other way.
TOLERANCE = {"float32": 1e-4, "bfloat16": 2e-2}
RUNS = [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16"), ("C", "float32"), ("C", "bfloat16")]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    made = {}
    for which in ("A", "B", "C"):
        made[(which, "bfloat16")] = tiny_configs.write_tiny(str(root / "bf16"), which, "bfloat16")
        made[(which, "float32")] = tiny_configs.write_tiny(str(root / "native"), which)
    return made


@pytest.fixture(scope="module")
def engines(folders):
    cache = {}

    def get(which, dtype, max_tokens=4096):
        key = (which, dtype, max_tokens)
        if key not in cache:
            cache[key] = engine_for(folders[(which, dtype)], dtype, "gpu", max_tokens)
        return cache[key]

    return get


def expected(folders, which, dtype, tokens):
    return plain_logits(folders[(which, dtype)], tokens, bf16=dtype == "bfloat16")


@pytest.mark.parametrize("which,dtype", RUNS)
def test_each_request_alone_and_whole(folders, engines, which, dtype):
    vocab = tiny_configs.CONFIGS[which]["vocab_size"]
    limit = tiny_configs.CONFIGS[which]["max_position_embeddings"]
    engine = engines(which, dtype)
    for tokens in random_prompts(vocab, [1, 2, 17, 64, 65, min(limit, 200)], seed=1):
        assert relative_error(run_whole(engine, tokens), expected(folders, which, dtype, tokens)) < TOLERANCE[dtype]
    engine.cache.check()


@pytest.mark.parametrize("which,dtype", RUNS)
def test_last_32_tokens_one_by_one(folders, engines, which, dtype):
    vocab = tiny_configs.CONFIGS[which]["vocab_size"]
    limit = tiny_configs.CONFIGS[which]["max_position_embeddings"]
    engine = engines(which, dtype)
    for tokens in random_prompts(vocab, [33, 100, min(limit, 130)], seed=2):
        wanted = expected(folders, which, dtype, tokens)[-32:]
        assert relative_error(run_tail_stepwise(engine, tokens, 32), wanted) < TOLERANCE[dtype]


@pytest.mark.parametrize("which,dtype", RUNS)
def test_unequal_batches_one_after_another(folders, engines, which, dtype):
    """Prompts of unequal lengths start together, shorter requests end earlier, and the next batch takes
    the slots and pages that the last one gave back."""
    vocab = tiny_configs.CONFIGS[which]["vocab_size"]
    engine = engines(which, dtype, 64 * 7)
    waves = {"A": ([5, 11, 17], 8), "B": ([1, 2, 9, 33, 64], 16), "C": ([70, 3, 130], 12)}
    prompt_lengths, steps = waves[which]
    for wave in range(3):
        lengths = prompt_lengths if wave != 1 else list(reversed(prompt_lengths))
        totals = [length + max(1, steps - 3 * index) for index, length in enumerate(lengths)]
        requests = random_prompts(vocab, totals, seed=20 + wave)
        found = run_batched(engine, requests, lengths)
        for request, length, logits in zip(requests, lengths, found):
            wanted = expected(folders, which, dtype, request)[length - 1 :]
            assert relative_error(logits, wanted) < TOLERANCE[dtype]
        engine.cache.check()
        assert engine.cache.slots.in_use == 0 and engine.cache.free_tokens() == 64 * 7


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, engines, dtype):
    """Hundreds of single-token steps across several pages."""
    engine = engines("C", dtype)
    (tokens,) = random_prompts(333, [400], seed=4)
    wanted = expected(folders, "C", dtype, tokens)[-390:]
    assert relative_error(run_tail_stepwise(engine, tokens, 390), wanted) < TOLERANCE[dtype]


@pytest.mark.parametrize("which,dtype", RUNS)
def test_first_tokens_of_a_sequence(folders, engines, which, dtype):
    """Position 0 alone, then positions 1 and 2 one by one: no earlier key exists."""
    vocab = tiny_configs.CONFIGS[which]["vocab_size"]
    engine = engines(which, dtype)
    (tokens,) = random_prompts(vocab, [3], seed=5)
    wanted = expected(folders, which, dtype, tokens)
    slot = engine.open_sequence()
    rows = [engine.step([StepEntry(slot, [token], [0])]).float().cpu().clone() for token in tokens]
    engine.close_sequence(slot)
    assert relative_error(torch.cat(rows), wanted) < TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_padding_and_neighbours_change_nothing(folders, engines, dtype):
    """A request's logits do not depend on what else is in the batch, beyond rounding.  In 32-bit the sums
    may only be ordered differently (1e-6).  In bfloat16 the number of rows picks another product kernel,
    whose sums round to bfloat16 the other way here and there, so the bound is the one of every other
    bfloat16 comparison."""
    engine = engines("B", dtype)
    requests = random_prompts(500, [40, 7, 64], seed=6)
    alone = run_batched(engine, requests[:1], [30])[0]
    beside = run_batched(engine, requests, [30, 3, 50])[0]
    assert relative_error(beside, alone) < (1e-6 if dtype == "float32" else TOLERANCE[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stale_pages_do_not_leak(folders, engines, dtype):
    """A long request fills pages with large values; a short one that reuses them must not see them."""
    engine = engines("A", dtype, 64 * 2)
    (long_request,) = random_prompts(256, [120], seed=7)
    run_whole(engine, long_request)
    for group in engine.cache.kv.values():   # poison what the finished request left behind
        group.keys.fill_(float("nan"))
        group.values.fill_(float("nan"))
    (short,) = random_prompts(256, [70], seed=8)
    found = run_tail_stepwise(engine, short, 5)
    assert torch.isfinite(found).all()
    assert relative_error(found, expected(folders, "A", dtype, short)[-5:]) < TOLERANCE[dtype]


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("B", "float32")])
def test_greedy_generation_through_the_entry_point(folders, which, dtype):
    """`generate()` on a folder: unequal prompts, more requests than one batch holds, the plain tokens."""
    config = plain_model.read_plain_config(folders[(which, dtype)])
    weights = plain_model.read_plain_weights(folders[(which, dtype)])
    lengths = {"A": [5, 11, 17, 3], "B": [1, 2, 9, 33, 64]}[which]
    steps = {"A": 8, "B": 16}[which]
    prompts = random_prompts(config.vocab_size, lengths, seed=9)
    output = generate(folders[(which, dtype)], prompts, max_new_tokens=steps, dtype=dtype, stop_tokens=(), max_batch=3)
    for prompt, result in zip(prompts, output):
        assert result.tokens == plain_model.greedy_generate(config, weights, prompt, steps)
        assert result.finish_reason == "length"
    assert output.metrics.batches == 2


def test_generation_stops_at_stop_tokens(folders):
    config = plain_model.read_plain_config(folders[("A", "float32")])
    weights = plain_model.read_plain_weights(folders[("A", "float32")])
    prompts = random_prompts(256, [6, 9], seed=10)
    free = [plain_model.greedy_generate(config, weights, prompt, 10) for prompt in prompts]
    stop = free[0][4]
    output = generate(folders[("A", "float32")], prompts, max_new_tokens=10, dtype="float32", stop_tokens=[stop])
    for run, result in zip(free, output):
        cut = run.index(stop) if stop in run else len(run)
        assert result.tokens == run[:cut]
        assert result.finish_reason == ("stop" if cut < len(run) else "length")


@pytest.mark.parametrize("dtype", ["bfloat16"])
def test_bfloat16_generation_follows_the_plain_ranking(folders, dtype):
    """In bfloat16 near-ties may fall the other way, so each chosen token must be (nearly) the plain best
    given the engine's own earlier tokens."""
    folder = folders[("B", dtype)]
    prompts = random_prompts(500, [9, 33], seed=11)
    output = generate(folder, prompts, max_new_tokens=8, dtype=dtype, stop_tokens=())
    for prompt, result in zip(prompts, output):
        assert len(result.tokens) == 8
        logits = plain_logits(folder, list(prompt) + result.tokens, bf16=True)
        for index, token in enumerate(result.tokens):
            row = logits[len(prompt) - 1 + index]
            assert float(row.max() - row[token]) <= TOLERANCE[dtype] * float(row.abs().max()) * 2


def test_temperature_sampling_is_repeatable(folders):
    folder = folders[("A", "bfloat16")]
    prompts = random_prompts(256, [5, 11, 17], seed=12)
    first = generate(folder, prompts, max_new_tokens=12, temperature=0.8, seed=3, stop_tokens=())
    again = generate(folder, prompts, max_new_tokens=12, temperature=0.8, seed=3, stop_tokens=())
    other = generate(folder, prompts, max_new_tokens=12, temperature=0.8, seed=4, stop_tokens=())
    assert [r.tokens for r in first] == [r.tokens for r in again]
    assert [r.tokens for r in first] != [r.tokens for r in other]


def test_same_request_twice_gives_the_same_tokens(folders):
    """crates/engine/src/qwen3_engine.rs:258-353 (the same chat twice gives identical output): the cache is reset."""
    folder = folders[("B", "bfloat16")]
    engine = engine_for(folder, "bfloat16", "gpu", 1024)
    prompts = random_prompts(500, [33], seed=13)
    first = generate(engine, prompts, max_new_tokens=16, stop_tokens=())
    second = generate(engine, prompts, max_new_tokens=16, stop_tokens=())
    assert first[0].tokens == second[0].tokens
    engine.cache.check()


@pytest.mark.parametrize("which,dtype", [("A", "bfloat16"), ("B", "bfloat16"), ("C", "float32")])
def test_plain_kernels_alone_give_the_same_logits(folders, which, dtype):
    """`--optimize-kernel false`: products by the tiled kernel, attention by the kernel over the pages, nothing fused.
    Whole prompts, the last tokens one by one, and an unequal batch, against the plain implementation and against the
    fast kernels: a fault that one of the two shows alone lies in a kernel, one that both show in the engine."""
    from tau_rs_b200.csrc import kernels

    vocab = tiny_configs.CONFIGS[which]["vocab_size"]
    limit = tiny_configs.CONFIGS[which]["max_position_embeddings"]
    (tokens,) = random_prompts(vocab, [min(limit, 120)], seed=41)
    requests = random_prompts(vocab, [40, 23, 9], seed=42)
    found = {}
    try:
        for optimized in (False, True):
            kernels.prefer_optimized(optimized)
            engine = engine_for(folders[(which, dtype)], dtype, "gpu", 1024)   # built under the setting: the feed-forward's weight layout follows it
            assert engine.model.blocks[0].feed_forward.fused == (optimized and dtype == "bfloat16")
            found[optimized] = (run_whole(engine, tokens), run_tail_stepwise(engine, tokens, 32), run_batched(engine, requests, [30, 3, 8]))
            engine.cache.check()
    finally:
        kernels.prefer_optimized(True)
    wanted = expected(folders, which, dtype, tokens)
    for optimized in (False, True):
        whole, tail, batched = found[optimized]
        assert relative_error(whole, wanted) < TOLERANCE[dtype]
        assert relative_error(tail, wanted[-32:]) < TOLERANCE[dtype]
        for request, prompt_length, logits in zip(requests, [30, 3, 8], batched):
            assert relative_error(logits, expected(folders, which, dtype, request)[prompt_length - 1 :]) < TOLERANCE[dtype]
    assert relative_error(found[False][0], found[True][0]) < TOLERANCE[dtype]


@pytest.mark.parametrize("which,dtype", [("A", "bfloat16"), ("C", "bfloat16"), ("B", "float32")])
@pytest.mark.parametrize("graphs", [True, False])
def test_a_given_attention_block_size_changes_no_logits(folders, which, dtype, graphs):
    """`--attention-block-size`: the context of a decode step cut into blocks of 32 or of 256 positions, whatever the batch."""
    vocab = tiny_configs.CONFIGS[which]["vocab_size"]
    limit = tiny_configs.CONFIGS[which]["max_position_embeddings"]
    (tokens,) = random_prompts(vocab, [min(limit, 200)], seed=43)
    wanted = expected(folders, which, dtype, tokens)[-32:]
    for block in (32, 256):
        engine = engine_for(folders[(which, dtype)], dtype, "gpu", 1024)
        engine.use_graphs = engine.use_graphs and graphs
        engine.attention_block_size = block
        assert engine.decode_splits(3, 200) == (8 if block == 32 else 1) and engine.decode_splits(1, 5000) == (64 if block == 32 else 32)
        assert relative_error(run_tail_stepwise(engine, tokens, 32), wanted) < TOLERANCE[dtype]


MEDIUM = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 5000, "hidden_size": 1024, "intermediate_size": 3072,
    "num_hidden_layers": 2, "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128, "attention_bias": False,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 2048, "tie_word_embeddings": True,
    "hidden_act": "silu", "torch_dtype": "bfloat16", "eos_token_id": 1,
}


OTHER_MEDIUM = dict(MEDIUM, vocab_size=3001, hidden_size=768, intermediate_size=2056, num_attention_heads=12, num_key_value_heads=4,
                    head_dim=64, attention_bias=True, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False)


@pytest.mark.parametrize("config", [MEDIUM, OTHER_MEDIUM], ids=["d128", "d64_bias_odd_vocab"])
def test_fast_kernels_against_plain_kernels_at_the_width_of_a_real_model(config):
    """The layer sizes of Qwen3-0.6B, and another set with heads of 64, biases, an intermediate width that is no multiple of 16
    and an odd vocabulary (two layers, a small vocabulary): the tiny configurations never reach the paired
    256 x 256 tiles, the products cut along K, the tensor-memory attention or clusters of decode blocks inside the engine.
    Prompts of 700 and 130 tokens, then decode batches of 1, 12 and 40 sequences; the plain kernels are the yardstick."""
    from tau_rs_b200 import Engine
    from tau_rs_b200.api import random_model
    from tau_rs_b200.csrc import kernels

    prompts = random_prompts(config["vocab_size"], [700, 130] + [70] * 38, seed=51)
    steps = 4
    found = {}
    try:
        for optimized in (False, True):
            kernels.prefer_optimized(optimized)
            engine = Engine(random_model(config, seed=9, dtype="bfloat16", norm_jitter=0.1), 64 * 128)
            rows = []
            for batch in ([0], list(range(1, 13)), list(range(40))):
                slots = [engine.open_sequence() for _ in batch]
                logits = engine.step([StepEntry(slot, prompts[i], [len(prompts[i]) - 1]) for slot, i in zip(slots, batch)])
                rows.append(logits.float().cpu())
                for step in range(steps):
                    tokens = [int(prompts[i][step]) for i in batch]           # given tokens, so that both runs feed the same
                    logits = engine.step([StepEntry(slot, [token], [0]) for slot, token in zip(slots, tokens)])
                    rows.append(logits.float().cpu())
                for slot in slots:
                    engine.close_sequence(slot)
                engine.cache.check()
            found[optimized] = rows
    finally:
        kernels.prefer_optimized(True)
    assert kernels.gemm_tc_status() == 0 and kernels.attention_prefill_tc_status(config["head_dim"]) == 0
    for fast, plain in zip(found[True], found[False]):
        assert fast.shape == plain.shape and torch.isfinite(fast).all()
        assert relative_error(fast, plain) < TOLERANCE["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_plain_implementation_at_the_width_of_a_real_model(tmp_path, dtype):
    """One layer of the second set of sizes above against the plain whole-sequence implementation, in 32-bit and in
    bfloat16: a prompt of 300 tokens whole, and its last 16 tokens one by one."""
    from tau_rs_b200.weights import write_random_model

    config = dict(OTHER_MEDIUM, num_hidden_layers=1, torch_dtype=dtype)
    folder = str(tmp_path / "medium")
    write_random_model(folder, config, seed=12, norm_jitter=0.1, storage=dtype)
    (tokens,) = random_prompts(config["vocab_size"], [300], seed=52)
    wanted = plain_logits(folder, tokens, bf16=dtype == "bfloat16")
    engine = engine_for(folder, dtype, "gpu", 1024)
    assert relative_error(run_whole(engine, tokens), wanted) < TOLERANCE[dtype]
    assert relative_error(run_tail_stepwise(engine, tokens, 16), wanted[-16:]) < TOLERANCE[dtype]
    engine.cache.check()


@pytest.mark.parametrize("length,config", [(5000, MEDIUM), (9000, OTHER_MEDIUM)], ids=["5000_d128", "9000_d64"])
def test_a_long_context_at_the_width_of_a_real_model(tmp_path, length, config):
    """One layer in bfloat16 over thousands of positions against the plain implementation: the prompt whole (dozens of
    query tiles and up to 141 key tiles of the tensor-memory attention; the first and the last row of every 64 are
    compared, each on its own), then six tokens one by one over a context that
    decode attention cuts into 16 blocks of one cluster (5,000 positions) or 32 that meet in global memory (9,000)."""
    from tau_rs_b200.csrc import kernels
    from tau_rs_b200.weights import write_random_model

    config = dict(config, num_hidden_layers=1, max_position_embeddings=16384, torch_dtype="bfloat16")
    folder = str(tmp_path / "long")
    write_random_model(folder, config, seed=13, norm_jitter=0.1, storage="bfloat16")
    (tokens,) = random_prompts(config["vocab_size"], [length + 6], seed=53)
    wanted = plain_logits(folder, tokens, bf16=True)
    engine = engine_for(folder, "bfloat16", "gpu", 64 * 160)
    assert engine.decode_splits(1, length + 1) == (16 if length <= 8192 else 32)
    slot = engine.open_sequence()
    places = sorted(set(list(range(0, length, 64)) + list(range(63, length, 64)) + [length // 2, length - 2, length - 1]))
    logits = engine.step([StepEntry(slot, tokens[:length], places)]).float().cpu()
    assert relative_error(logits, wanted[places]) < TOLERANCE["bfloat16"]
    for row, place in enumerate(places):     # row by row: one query tile's lost keys must not hide behind another row's largest logit
        assert relative_error(logits[row], wanted[place]) < TOLERANCE["bfloat16"], place
    for index in range(length, length + 6):
        logits = engine.step([StepEntry(slot, [tokens[index]], [0])]).float().cpu()
        assert relative_error(logits, wanted[index : index + 1]) < TOLERANCE["bfloat16"]
    engine.close_sequence(slot)
    engine.cache.check()
    assert kernels.attention_prefill_tc_status(config["head_dim"]) == 0 and kernels.gemm_tc_status() == 0


def test_a_cache_larger_than_the_device_is_refused_before_anything_is_allocated(folders):
    """crates/engine/src/model_engine/kv_budget.rs:17-56: a named error, not an out-of-memory failure of the allocator."""
    from tau_rs_b200 import CacheDoesNotFit, Engine, load_model

    model = load_model(folders[("A", "float32")], "float32", "gpu")
    free, total = torch.cuda.mem_get_info()
    before = torch.cuda.memory_allocated()
    per_token = 2 * 2 * 2 * 16 * 4          # keys and values, 2 layers, 2 KV heads of 16, 32-bit
    with pytest.raises(CacheDoesNotFit) as refusal:
        Engine(model, max_tokens=(total // per_token) * 2)
    assert torch.cuda.memory_allocated() == before
    assert 0 < refusal.value.fitting_tokens < total // per_token and "fits" in str(refusal.value)
    engine = Engine(model, max_tokens=4096, headroom_bytes=0)
    assert engine.capacity_tokens == 4096
