"""Ways of cutting the work that the other tests do not run: a prompt that enters the cache in chunks through the
tensor-memory attention, a step that mixes a run of tokens with single tokens, the generation loop in bfloat16 with
chunks, several batches and a stop token, and the command line as a subprocess."""
import hashlib
import json
import os
import subprocess

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs
from helpers import engine_for, plain_logits, random_prompts, relative_error
from tau_rs_b200 import StepEntry, generate
from tau_rs_b200.weights import write_random_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOLERANCE = {"float32": 1e-4, "bfloat16": 2e-2}

# Head sizes that the tensor-memory attention serves, at widths that the plain implementation walks through in seconds.
HEADS_128 = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 1000, "hidden_size": 256, "intermediate_size": 512,
    "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "attention_bias": False,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 1024, "tie_word_embeddings": True, "hidden_act": "silu",
    "eos_token_id": 1,
}
HEADS_64 = dict(HEADS_128, vocab_size=777, hidden_size=192, intermediate_size=328, num_attention_heads=6, num_key_value_heads=1, head_dim=64,
                attention_bias=True, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, num_hidden_layers=3)
CONFIGS = {"d128": HEADS_128, "d64": HEADS_64}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("schedules")
    made = {}
    for name, config in CONFIGS.items():
        for dtype in ("float32", "bfloat16"):
            made[(name, dtype)] = str(root / f"{name}_{dtype}")
            write_random_model(made[(name, dtype)], config, seed=31, norm_jitter=0.1, storage=dtype)
    for dtype in ("float32", "bfloat16"):
        made[("A", dtype)] = tiny_configs.write_tiny(str(root / dtype), "A", dtype)
    return made


@pytest.mark.parametrize("name", ["d128", "d64"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_in_chunks_of_100_tokens(folders, name, dtype):
    """Every chunk after the first is a run of new tokens behind cached ones (crates/engine/src/model_engine/tests/
    generation.rs:48-125 checks the offsets of such chunks; here their logits)."""
    from tau_rs_b200.csrc import kernels

    folder = folders[(name, dtype)]
    (tokens,) = random_prompts(CONFIGS[name]["vocab_size"], [470], seed=71)
    wanted = plain_logits(folder, tokens, bf16=dtype == "bfloat16")
    engine = engine_for(folder, dtype, "gpu", 1024)
    slot = engine.open_sequence()
    found = []
    for begin in range(0, len(tokens), 100):
        piece = tokens[begin : begin + 100]
        found.append(engine.step([StepEntry(slot, piece, list(range(len(piece))))]).float().cpu().clone())
    engine.close_sequence(slot)
    found = torch.cat(found)
    assert relative_error(found, wanted) < TOLERANCE[dtype]
    for row in (99, 100, 101, 199, 200, 399, 400, 469):
        assert relative_error(found[row], wanted[row]) < TOLERANCE[dtype], row
    engine.cache.check()
    assert kernels.attention_prefill_tc_status(CONFIGS[name]["head_dim"]) == 0 and kernels.gemm_tc_status() == 0


@pytest.mark.parametrize("name", ["d128", "d64"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_that_mixes_a_run_with_single_tokens(folders, name, dtype):
    """One sequence brings 70 tokens behind 30 cached ones, three others one token each behind contexts of unequal
    lengths, in one step; then all four bring one token."""
    folder = folders[(name, dtype)]
    requests = random_prompts(CONFIGS[name]["vocab_size"], [101, 66, 130, 3], seed=72)
    held = [30, 64, 128, 1]
    engine = engine_for(folder, dtype, "gpu", 1024)
    slots = [engine.open_sequence() for _ in requests]
    engine.step([StepEntry(slot, request[:count], []) for slot, request, count in zip(slots, requests, held)])
    mixed = engine.step([StepEntry(slots[0], requests[0][30:100], [0, 34, 69])] +
                        [StepEntry(slot, [request[count]], [0]) for slot, request, count in list(zip(slots, requests, held))[1:]])
    mixed = mixed.float().cpu().clone()
    after = [100, 65, 129, 2]
    single = engine.step([StepEntry(slot, [request[count]], [0]) for slot, request, count in zip(slots, requests, after)]).float().cpu().clone()
    for slot in slots:
        engine.close_sequence(slot)
    plain = [plain_logits(folder, request, bf16=dtype == "bfloat16") for request in requests]
    wanted_mixed = torch.stack([plain[0][30], plain[0][64], plain[0][99], plain[1][64], plain[2][128], plain[3][1]])
    wanted_single = torch.stack([plain[0][100], plain[1][65], plain[2][129], plain[3][2]])
    for row in range(6):
        assert relative_error(mixed[row], wanted_mixed[row]) < TOLERANCE[dtype], row
    for row in range(4):
        assert relative_error(single[row], wanted_single[row]) < TOLERANCE[dtype], row
    engine.cache.check()


def test_generation_in_bfloat16_with_chunks_batches_and_a_stop_token(folders):
    """`generate(prefill_chunk_tokens=64)` with five requests in batches of two: the same call twice gives the same tokens;
    every chosen token is (nearly) the plain best given the engine's own earlier tokens; with one of the produced tokens
    as stop token every request ends where that token first came."""
    folder = folders[("d128", "bfloat16")]
    prompts = random_prompts(1000, [150, 9, 70, 129, 33], seed=73)
    engine = engine_for(folder, "bfloat16", "gpu", 64 * 8)
    free = generate(engine, prompts, max_new_tokens=10, stop_tokens=(), max_batch=2, prefill_chunk_tokens=64)
    again = generate(engine, prompts, max_new_tokens=10, stop_tokens=(), max_batch=2, prefill_chunk_tokens=64)
    assert [result.tokens for result in free] == [result.tokens for result in again]
    assert free.metrics.batches == 3 and free.metrics.prefill_steps >= 3 + 1 + 1
    for prompt, result in zip(prompts, free):
        assert len(result.tokens) == 10 and result.finish_reason == "length"
        logits = plain_logits(folder, list(prompt) + result.tokens, bf16=True)
        for index, token in enumerate(result.tokens):
            row = logits[len(prompt) - 1 + index]
            assert float(row.max() - row[token]) <= 2 * TOLERANCE["bfloat16"] * float(row.abs().max())
    stop = free[2].tokens[4]
    stopped = generate(engine, prompts, max_new_tokens=10, stop_tokens=[stop], max_batch=2, prefill_chunk_tokens=64)
    for run, result in zip(free, stopped):
        cut = run.tokens.index(stop) if stop in run.tokens else len(run.tokens)
        assert result.tokens == run.tokens[:cut]
        assert result.finish_reason == ("stop" if cut < len(run.tokens) else "length")
    engine.cache.check()
    assert engine.cache.slots.in_use == 0


def test_temperature_sampling_does_not_depend_on_the_batch(folders):
    """Request numbers key the noise, so a request that is number 0 of its call draws the same tokens alone, beside two
    others, and in a batch of its own (32-bit, where the logits do not depend on the batch beyond 1e-6)."""
    folder = folders[("A", "float32")]
    prompts = random_prompts(256, [11, 5, 17], seed=12)
    beside = generate(folder, prompts, max_new_tokens=12, temperature=0.8, seed=3, stop_tokens=(), dtype="float32")
    alone = generate(folder, prompts[:1], max_new_tokens=12, temperature=0.8, seed=3, stop_tokens=(), dtype="float32")
    one_by_one = generate(folder, prompts, max_new_tokens=12, temperature=0.8, seed=3, stop_tokens=(), dtype="float32", max_batch=1)
    assert alone[0].tokens == beside[0].tokens and len(alone[0].tokens) == 12
    assert [result.tokens for result in one_by_one] == [result.tokens for result in beside]
    greedy = generate(folder, prompts[:1], max_new_tokens=12, stop_tokens=(), dtype="float32")
    assert greedy[0].tokens != alone[0].tokens


# ---- the command line -------------------------------------------------------------------------------------------------
def run_cli(arguments):
    done = subprocess.run([os.path.join(ROOT, "bin", "tau")] + arguments, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    records = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    trace = [json.loads(line[len("inference_trace "):]) for line in done.stdout.splitlines() if line.startswith("inference_trace ")]
    return records, trace, done.stderr


def test_the_command_line_generates_the_plain_tokens(folders, tmp_path):
    """`bin/tau` on a folder, greedy, in 32-bit: the plain implementation's tokens, with graphs and without; the trace's
    hash of the prompt step's logits is the hash of what `bin/trace_run` writes for the same step
    (crates/engine/src/model_engine/tests/gpu_generation.rs:106-172: a traced generation equals an ordinary one)."""
    folder = folders[("A", "float32")]
    config = plain_model.read_plain_config(folder)
    weights = plain_model.read_plain_weights(folder)
    prompts = random_prompts(256, [9, 4], seed=74)
    wanted = [plain_model.greedy_generate(config, weights, prompt, 7, stop_tokens=(7,)) for prompt in prompts]
    base = ["--model", folder, "--device", "gpu", "--dtype", "f32", "--max-tokens", "7"]
    for prompt in prompts:
        base += ["--prompt-ids", ",".join(str(token) for token in prompt)]
    records, _, _ = run_cli(base)
    assert [record["tokens"] for record in records] == wanted
    assert [record["finish_reason"] for record in records] == ["length" if len(tokens) == 7 else "stop" for tokens in wanted]
    records, trace, errors = run_cli(base + ["--cuda-graph", "none", "--tracing", "--metrics", "--vram-metrics", "--hbm-gbs", "6537.3"])
    assert [record["tokens"] for record in records] == wanted
    report = [json.loads(line[len("inference_metrics "):]) for line in errors.splitlines() if line.startswith("inference_metrics ")][-1]
    assert report["status"] == "ok" and report["decode_tokens"] > 0 and report["decode_gb_per_second"] > 0
    assert report["fraction_of_roofline"] is not None and 0 <= report["fraction_of_roofline"] < 1   # a tiny model reads next to nothing
    (trace,) = trace
    assert trace["generated"] == wanted and trace["prompts"] == prompts
    first = [step for step in trace["steps"] if step["request"] == 0 and step["phase"] == "prefill"][0]
    assert first["cache_offset"] == 0 and first["input_tokens"] == 9 and first["token_id"] == wanted[0][0] and first["is_eos"] is False
    assert len(first["logits"]["samples"]) == 16 and first["logits"]["count"] == 256 and first["duration_us"] > 0
    assert set(first["kernel_class_ms"]) >= {"embedding", "norm", "product", "attention"} and first["kernel_class_ms"]["product"] > 0
    decode = [step for step in trace["steps"] if step["request"] == 0 and step["phase"] == "decode"]
    assert [step["cache_offset"] for step in decode] == [9 + index for index in range(len(decode))]
    out = tmp_path / "replay"
    lines = "".join(json.dumps(step) + "\n" for step in (
        {"step": 0, "entries": [{"id": "a", "tokens": prompts[0], "want": [8]}, {"id": "b", "tokens": prompts[1], "want": [3]}], "end": ["a", "b"]},))
    done = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                          input=lines, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    replayed = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, 256)
    assert hashlib.sha256(replayed[0].tobytes()).hexdigest() == first["logits"]["sha256_f32_le"]


def test_the_command_line_in_bfloat16_with_a_temperature(folders):
    folder = folders[("A", "bfloat16")]
    arguments = ["-m", folder, "--dtype", "bf16", "--max-tokens", "9", "--temperature", "0.7", "--seed", "5", "--stop-ids", "",
                 "--prompt-ids", "5,17,3,200,9", "--prompt-ids", "1 2 3", "--attention-block-size", "32", "--prefill-chunk-size", "4"]
    first, _, _ = run_cli(arguments)
    second, _, _ = run_cli(arguments)
    assert [record["tokens"] for record in first] == [record["tokens"] for record in second]
    assert all(len(record["tokens"]) == 9 and record["finish_reason"] == "length" for record in first)
    other, _, _ = run_cli(arguments[:9] + ["6"] + arguments[10:])
    assert [record["tokens"] for record in other] != [record["tokens"] for record in first]
