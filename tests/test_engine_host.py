"""The engine's host logic on the CPU, with the kernels replaced by their plain torch statements.

What is tested here is packing, page and slot bookkeeping, the schedule and the cache
addressing, in every way of cutting the work; the CUDA kernels themselves are tested on the
GPU.  Expected logits come from the plain whole-sequence implementation.
"""
import pytest
import torch

import plain_kernels
import tiny_configs
from helpers import (engine_for, plain_logits, random_prompts, relative_error, run_batched, run_tail_stepwise, run_whole)
from tau_rs_b200 import CacheFull, StepEntry, StepError


@pytest.fixture
def cpu_kernels(monkeypatch):
    plain_kernels.install(monkeypatch)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {which: tiny_configs.write_tiny(str(root), which) for which in ("A", "B", "C")}


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_whole_prompt_matches_plain(cpu_kernels, folders, which):
    vocab = tiny_configs.CONFIGS[which]["vocab_size"]
    engine = engine_for(folders[which], "float32", "cpu")
    for tokens in random_prompts(vocab, [1, 17, 70], seed=5):
        assert relative_error(run_whole(engine, tokens), plain_logits(folders[which], tokens)) < 1e-4
    engine.cache.check()


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_tail_stepwise_matches_whole(cpu_kernels, folders, which):
    vocab = tiny_configs.CONFIGS[which]["vocab_size"]
    engine = engine_for(folders[which], "float32", "cpu")
    (tokens,) = random_prompts(vocab, [100], seed=6)
    wanted = plain_logits(folders[which], tokens)[-32:]
    assert relative_error(run_tail_stepwise(engine, tokens, 32), wanted) < 1e-4


@pytest.mark.parametrize("which", ["A", "B"])
def test_unequal_batches_reuse_slots(cpu_kernels, folders, which):
    vocab = tiny_configs.CONFIGS[which]["vocab_size"]
    engine = engine_for(folders[which], "float32", "cpu", max_tokens=64 * 6)
    lengths = [[5, 11, 17], [70, 3, 64, 1], [9, 65]]
    steps = [8, 3, 16]
    for wave, (prompt_lengths, extra) in enumerate(zip(lengths, steps)):
        totals = [length + (extra if index % 2 == 0 else extra // 2) for index, length in enumerate(prompt_lengths)]
        requests = random_prompts(vocab, totals, seed=10 + wave)
        found = run_batched(engine, requests, prompt_lengths)
        for request, prompt_length, logits in zip(requests, prompt_lengths, found):
            wanted = plain_logits(folders[which], request)[prompt_length - 1 :]
            assert logits.shape == wanted.shape
            assert relative_error(logits, wanted) < 1e-4
        engine.cache.check()
        assert engine.cache.slots.in_use == 0


def test_bfloat16_rounding_points_match_plain(cpu_kernels, folders):
    engine = engine_for(folders["A"], "bfloat16", "cpu")
    (tokens,) = random_prompts(256, [40], seed=3)
    wanted = plain_logits(folders["A"], tokens, bf16=True)
    assert relative_error(run_whole(engine, tokens), wanted) < 2e-2


def test_step_refuses_bad_entries(cpu_kernels, folders):
    engine = engine_for(folders["A"], "float32", "cpu", max_tokens=128)
    slot = engine.open_sequence()
    with pytest.raises(StepError):
        engine.step([])
    with pytest.raises(StepError):
        engine.step([StepEntry(slot, [], [])])
    with pytest.raises(StepError):
        engine.step([StepEntry(slot, [1, 2], [2])])
    with pytest.raises(StepError):
        engine.step([StepEntry(slot, [256], [0])])
    with pytest.raises(StepError):
        engine.step([StepEntry(slot, [1], [0]), StepEntry(slot, [2], [0])])
    with pytest.raises(StepError):
        engine.step([StepEntry(slot + 1, [1], [0])])
    with pytest.raises(CacheFull):
        engine.step([StepEntry(slot, list(range(129)), [0])])   # beyond max_position_embeddings
    other = engine.open_sequence()
    with pytest.raises(CacheFull):
        engine.step([StepEntry(slot, list(range(100)), [0]), StepEntry(other, list(range(60)), [0])])  # 3 pages wanted, 2 exist
    assert engine.sequence_length(slot) == 0 and engine.sequence_length(other) == 0
    engine.cache.check()
    assert engine.cache.free_tokens() == 128
    assert engine.step([StepEntry(slot, [1, 2, 3], [])]) is None
    assert engine.sequence_length(slot) == 3


def test_generation_one_step_ahead_equals_step_by_step(cpu_kernels, folders):
    """`generate` through the engine and the sampler's two halves (decoding one step ahead of the host) against the same
    loop with a plain `select` function: stop tokens in the middle, unequal limits, more requests than one batch holds."""
    from tau_rs_b200 import Sampler
    from tau_rs_b200.engine import generate_tokens

    vocab = tiny_configs.CONFIGS["A"]["vocab_size"]
    prompts = random_prompts(vocab, [5, 1, 33, 70, 9], seed=21)
    limits = [12, 1, 7, 20, 3]
    sampler = Sampler()
    step_by_step = generate_tokens(engine_for(folders["A"], "float32", "cpu", max_tokens=64 * 6), prompts, limits,
                                   lambda logits, requests, indices: sampler.select(logits, requests, indices), max_batch=3)
    for stop in ((), tuple(step_by_step[3].tokens[4:6])):
        plain = generate_tokens(engine_for(folders["A"], "float32", "cpu", max_tokens=64 * 6), prompts, limits,
                                lambda logits, requests, indices: sampler.select(logits, requests, indices), stop_tokens=stop, max_batch=3)
        engine = engine_for(folders["A"], "float32", "cpu", max_tokens=64 * 6)
        ahead = generate_tokens(engine, prompts, limits, sampler, stop_tokens=stop, max_batch=3)
        assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in plain]
        engine.cache.check()


def test_step_takes_token_ids_from_the_device_or_refuses_them(cpu_kernels, folders):
    vocab = tiny_configs.CONFIGS["B"]["vocab_size"]
    (tokens,) = random_prompts(vocab, [20], seed=8)
    wanted = plain_logits(folders["B"], tokens)
    engine = engine_for(folders["B"], "float32", "cpu")
    slot = engine.open_sequence()
    engine.step([StepEntry(slot, tokens[:19], [])])
    # The id comes from a tensor; the entry's own token is a placeholder.
    logits = engine.step([StepEntry(slot, [0], [0])], device_tokens=torch.tensor([tokens[19]], dtype=torch.int32))
    assert relative_error(logits, wanted[19:20]) < 1e-4
    length = engine.sequence_length(slot)
    for entries, ids in (([StepEntry(slot, [0, 0], [1])], torch.tensor([1, 2], dtype=torch.int32)),      # two tokens in one entry
                         ([StepEntry(slot, [0], [0])], torch.tensor([1, 2], dtype=torch.int32)),          # one id too many
                         ([StepEntry(slot, [0], [0])], torch.tensor([1], dtype=torch.int64))):            # not int32
        with pytest.raises(StepError):
            engine.step(entries, device_tokens=ids)
        assert engine.sequence_length(slot) == length      # refused before anything changed
    engine.close_sequence(slot)
    engine.cache.check()


def test_windowed_layers_give_pages_back_and_lose_nothing(cpu_kernels, tmp_path):
    from helpers import WINDOW_CONFIG, window_spec, windowed_cache_matches_whole_prompt
    from tau_rs_b200 import write_random_model
    from tau_rs_b200.config import register_architecture, unregister_architecture

    register_architecture("ToyWindowForCausalLM", "toy_window", lambda raw: raw, window_spec)
    try:
        folder = str(tmp_path / "window")
        write_random_model(folder, WINDOW_CONFIG, seed=9, norm_jitter=0.1, storage="float32")
        windowed_cache_matches_whole_prompt(folder, "float32", torch.device("cpu"), 1e-4)
    finally:
        unregister_architecture("ToyWindowForCausalLM")


def test_generation_plans_windowed_requests_by_what_they_hold_at_once(cpu_kernels, tmp_path):
    """Where every group of keys and values has a window, a request holds about a window and one run of pages however long
    it grows: the generation loop runs requests of up to 500 tokens through a cache of 9 pages (576 positions), two at a time, and
    gives the tokens that a roomy cache gives.  Without a window the same plan is refused."""
    from helpers import WINDOW_CONFIG, window_spec
    from tau_rs_b200 import Engine, generate, load_model, write_random_model
    from tau_rs_b200.config import register_architecture, unregister_architecture

    register_architecture("ToyWindowForCausalLM", "toy_window", lambda raw: raw, window_spec)
    try:
        folder = str(tmp_path / "window")
        write_random_model(folder, WINDOW_CONFIG, seed=9, norm_jitter=0.1, storage="float32")
        model = load_model(folder, "float32", torch.device("cpu"))
        prompts = random_prompts(WINDOW_CONFIG["vocab_size"], [400, 30, 260], seed=14)
        roomy = generate(Engine(model, 64 * 40), prompts, max_new_tokens=100, stop_tokens=(), prefill_chunk_tokens=32)
        tight_engine = Engine(model, 64 * 9)
        assert tight_engine.peak_cache_tokens(400, 500, 32) == 70 + 32 + 3 * 64 and tight_engine.peak_cache_tokens(400, 500) == 500
        assert tight_engine.peak_cache_tokens(30, 130, 32) == 130
        tight = generate(tight_engine, prompts, max_new_tokens=100, stop_tokens=(), prefill_chunk_tokens=32, max_batch=2)
        assert [result.tokens for result in tight] == [result.tokens for result in roomy]
        assert tight.metrics.batches == 2
        tight_engine.cache.check()
        assert tight_engine.cache.slots.in_use == 0 and tight_engine.cache.free_tokens() == 64 * 9
        with pytest.raises(ValueError, match="cache tokens"):
            generate(Engine(model, 64 * 6), prompts, max_new_tokens=100, stop_tokens=())      # whole prompts in one run: 500 positions do not fit 384
    finally:
        unregister_architecture("ToyWindowForCausalLM")
