"""The engine at the widths that are benchmarked, against the plain whole-sequence implementation.

Two layers of the Qwen3-8B sizes (hidden 4096, 32 query and 8 KV heads of 128, intermediate 12288, vocabulary 151936,
untied head) and the whole depth of the Qwen3-0.6B sizes (28 layers, tied head), with random weights drawn on the GPU;
the plain implementation gets the same values on the CPU.  The tiny configurations never meet the products with a
depth of 12288, the gated product of 24576 rows, the head of 151936 rows through the tensor-core kernel (a batch of
64) or through the skinny kernel's thousands of blocks (a batch of 8), or 28 layers of accumulated rounding.
The shape of the checks follows the reference's own numerics fixtures (crates/models/src/qwen3_5.rs:258-310: one
prefill and one cached decode step against stored values with a stated tolerance).
"""
import numpy as np
import pytest
import torch

import plain_model
from helpers import drawn_models, plain_rows, random_prompts, relative_error, run_batched
from tau_rs_b200 import Engine, StepEntry, generate

pytestmark = pytest.mark.gpu
TOLERANCE = {"float32": 1e-4, "bfloat16": 2e-2}
DTYPES = ["float32", "bfloat16"]

WIDE_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "attention_bias": False,
    "max_position_embeddings": 4096, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
DEEP_06B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 28, "hidden_size": 1024,
    "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 3072, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "attention_bias": False,
    "max_position_embeddings": 2048, "hidden_act": "silu", "torch_dtype": "bfloat16",
}


class Drawn:
    """A drawn model in both dtypes with one engine each, and the plain implementation's rows, kept once computed."""

    def __init__(self, config, seed, cache_tokens):
        self.vocab = config["vocab_size"]
        self.plain_config, self.plain_weights, self.models = drawn_models(config, seed, 0.1, DTYPES)
        self.engines = {dtype: Engine(model, cache_tokens) for dtype, model in self.models.items()}
        self._known = {}

    def plain(self, tokens, rows, dtype):
        key = (tuple(tokens), tuple(rows), dtype)
        if key not in self._known:
            self._known[key] = plain_rows(self.plain_config, self.plain_weights, list(tokens), list(rows), dtype == "bfloat16")
        return self._known[key]


@pytest.fixture(scope="module")
def wide():
    drawn = Drawn(WIDE_8B, seed=21, cache_tokens=64 * 96)
    yield drawn
    drawn.engines.clear()
    drawn.models.clear()
    torch.cuda.empty_cache()


@pytest.fixture(scope="module")
def deep():
    drawn = Drawn(DEEP_06B, seed=22, cache_tokens=64 * 128)
    yield drawn
    drawn.engines.clear()
    drawn.models.clear()
    torch.cuda.empty_cache()


def no_wait_ran_out(head_dim=128):
    from tau_rs_b200.csrc import kernels

    assert kernels.gemm_tc_status() == 0 and kernels.attention_prefill_tc_status(head_dim) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_whole_and_its_last_32_tokens_one_by_one(wide, dtype):
    engine = wide.engines[dtype]
    (tokens,) = random_prompts(wide.vocab, [300], seed=61)
    places = [0, 1, 63, 64, 127, 128, 255] + list(range(268, 300))
    wanted = wide.plain(tokens, places, dtype)
    slot = engine.open_sequence()
    whole = engine.step([StepEntry(slot, tokens, places)]).float().cpu().clone()
    engine.close_sequence(slot)
    assert relative_error(whole, wanted) < TOLERANCE[dtype]
    slot = engine.open_sequence()
    engine.step([StepEntry(slot, tokens[:268], [])])
    tail = torch.cat([engine.step([StepEntry(slot, [token], [0])]).float().cpu().clone() for token in tokens[268:]])
    engine.close_sequence(slot)
    assert relative_error(tail, wanted[7:]) < TOLERANCE[dtype]
    # Row by row as well: one wrong row among 32 must not hide behind the largest logit of another.
    for row in range(32):
        assert relative_error(tail[row], wanted[7 + row]) < TOLERANCE[dtype], row
    engine.cache.check()
    no_wait_ran_out()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_that_shrink_one_after_another(wide, dtype):
    engine = wide.engines[dtype]
    for wave, lengths in enumerate(([130, 70, 200], [9, 190, 64])):
        totals = [length + extra for length, extra in zip(lengths, (6, 3, 1))]
        requests = random_prompts(wide.vocab, totals, seed=62 + wave)
        found = run_batched(engine, requests, lengths)
        for request, length, logits in zip(requests, lengths, found):
            wanted = wide.plain(request, range(length - 1, len(request)), dtype)
            assert relative_error(logits, wanted) < TOLERANCE[dtype]
        engine.cache.check()
        assert engine.cache.slots.in_use == 0
    no_wait_ran_out()


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_batches_of_64_and_of_8(wide, dtype):
    """64 short prompts start together; two steps of 64 single tokens (the tensor-core products cut along K, the head
    through the tensor-core kernel with 32-bit output); then 56 requests end and 8 go on for two steps (the skinny
    products, the head over thousands of blocks)."""
    engine = wide.engines[dtype]
    lengths = [3 + (7 * index) % 18 for index in range(64)]
    requests = random_prompts(wide.vocab, [length + 4 for length in lengths], seed=64)
    slots = [engine.open_sequence() for _ in requests]
    found = [[] for _ in requests]
    logits = engine.step([StepEntry(slot, request[:length], [length - 1]) for slot, request, length in zip(slots, requests, lengths)])
    for index, row in enumerate(logits.float().cpu()):
        found[index].append(row.clone())
    live = list(range(64))
    for step in range(4):
        if step == 2:
            for index in live[8:]:
                engine.close_sequence(slots[index])
            live = live[:8]
        logits = engine.step([StepEntry(slots[index], [requests[index][lengths[index] + step]], [0]) for index in live])
        for index, row in zip(live, logits.float().cpu()):
            found[index].append(row.clone())
    for index in live:
        engine.close_sequence(slots[index])
    engine.cache.check()
    for index, (request, length) in enumerate(zip(requests, lengths)):
        rows = torch.stack(found[index])
        wanted = wide.plain(request, range(length - 1, length - 1 + rows.shape[0]), dtype)
        assert relative_error(rows, wanted) < TOLERANCE[dtype], index
    no_wait_ran_out()


def test_a_prefill_of_2048_tokens_in_bfloat16_against_the_32_bit_path(wide):
    """The benchmark's prefill: the paired 256 x 256 tiles over 2,048 tokens, the tensor-memory attention over 16 query
    tiles; the yardstick is the engine's own 32-bit path, which the tests above tie to the plain implementation."""
    (tokens,) = random_prompts(wide.vocab, [2048], seed=65)
    places = [0, 255, 256, 1023, 1024, 2046, 2047]
    rows = {}
    for dtype in DTYPES:
        engine = wide.engines[dtype]
        slot = engine.open_sequence()
        rows[dtype] = engine.step([StepEntry(slot, tokens, places)]).float().cpu().clone()
        engine.close_sequence(slot)
    for row in range(len(places)):
        assert relative_error(rows["bfloat16"][row], rows["float32"][row]) < TOLERANCE["bfloat16"], places[row]
    no_wait_ran_out()


# ---- the whole depth of the 0.6B sizes --------------------------------------------------------------------------------
def workload_prompts(vocab):
    """16 prompts with lengths uniform in [1, 1024] from seed 3, token ids uniform."""
    lengths = np.random.default_rng(3).integers(1, 1025, size=16).tolist()
    return random_prompts(vocab, lengths, seed=3)


def test_28_layers_in_32_bit_against_the_plain_implementation(deep):
    prompts = sorted(workload_prompts(deep.vocab), key=len)[:3]
    engine = deep.engines["float32"]
    for prompt in prompts:
        places = [0, len(prompt) // 2, len(prompt) - 1]
        wanted = deep.plain(prompt, places, "float32")
        slot = engine.open_sequence()
        found = engine.step([StepEntry(slot, prompt, places)]).float().cpu().clone()
        engine.close_sequence(slot)
        assert relative_error(found, wanted) < TOLERANCE["float32"]


def test_greedy_generation_of_the_unequal_batch_of_16(deep):
    """`generate()` over the 16 prompts at once in 32-bit; the three shortest requests must give the plain
    implementation's greedy tokens, which recomputes the whole sequence for every token.  In bfloat16 every chosen token
    must be (nearly) the plain best given the engine's own earlier tokens."""
    prompts = workload_prompts(deep.vocab)
    steps = 6
    output = generate(deep.engines["float32"], prompts, max_new_tokens=steps, stop_tokens=())
    assert [len(result.tokens) for result in output] == [steps] * 16
    shortest = sorted(range(16), key=lambda index: len(prompts[index]))[:3]
    for index in shortest:
        assert output[index].tokens == plain_model.greedy_generate(deep.plain_config, deep.plain_weights, prompts[index], steps)
    output = generate(deep.engines["bfloat16"], prompts, max_new_tokens=steps, stop_tokens=())
    for index in shortest:
        tokens = list(prompts[index]) + output[index].tokens
        places = range(len(prompts[index]) - 1, len(tokens) - 1)
        logits = deep.plain(tokens, places, "bfloat16")
        for row, token in zip(logits, output[index].tokens):
            assert float(row.max() - row[token]) <= 2 * TOLERANCE["bfloat16"] * float(row.abs().max())
    deep.engines["bfloat16"].cache.check()
    no_wait_ran_out()
