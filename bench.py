"""Decode and prefill throughput of dense Qwen3 shapes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--shape 8b|0.6b|32b]

Prints one JSON line.  The default run is the Qwen3-8B shape: `value` is decoded tokens per second at batch 8
with 2,048-token prompts (a step is one decode step of the whole batch), timed on the device with CUDA events around
exactly K steps; `e2e` is the same through `tau_rs_b200.generate` with host tokens in and out of every step (one call:
the prompts, W untimed decode steps, then K timed ones, read off the metrics that the call keeps at every token boundary);
`prefill` is one 2,048-token prompt; `points` are batch 1 and 64.  `--shape 0.6b` runs that shape's workload (16
prompts with lengths uniform in [1, 1024] from seed 3, then greedy and temperature-0.8 decoding), `--shape 32b` its own
(32 prompts of 4,096 tokens that enter the cache in chunks, then decoding).  The weights are far larger than L2 in
every shape, so nothing is flushed between decode steps.

`--impl reference`: taurs-ai/tau.rs cannot be built here, so there is no end-to-end number; what can run of it are four
generic kernels (see baseline/build_ref.py), which this arm times at the benchmark's sizes, without loading anything
of this library.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def qwen3(layers, hidden, heads, kv_heads, intermediate, tied):
    return {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": layers, "hidden_size": hidden,
        "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": 128, "intermediate_size": intermediate,
        "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": tied, "attention_bias": False,
        "max_position_embeddings": 40960, "hidden_act": "silu", "torch_dtype": "bfloat16",
    }


# name -> (config, batch, prompt tokens (0: unequal, uniform in [1, 1024] from seed 3), default steps, prefill chunk over the batch)
SHAPES = {
    "8b": (qwen3(36, 4096, 32, 8, 12288, False), 8, 2048, 64, 0),
    "0.6b": (qwen3(28, 1024, 16, 8, 3072, True), 16, 0, 128, 0),
    "32b": (qwen3(64, 5120, 64, 8, 25600, False), 32, 4096, 256, 8192),
}
SLOTS_PER_SEQUENCE = 8192


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as handle:
            raw = json.load(handle)
        return {"hbm_gbs": raw["hbm_gbs"], "bf16_tflops": raw["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.process = [], None

    def start(self):
        try:
            self.process = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.process = None

    def _read(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        clocks, peak, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [part.strip() for part in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                clocks.append(float(parts[0]))
                peak = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[2:]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": peak, "reasons": sorted(reasons),
                "samples": len(clocks)}


def prefill_flops(config, layers, lengths):
    """Products of every token and attention over the causal half of every prompt; the head at one row per prompt."""
    h, i, d = config["hidden_size"], config["intermediate_size"], config["head_dim"]
    nq, nkv = config["num_attention_heads"], config["num_key_value_heads"]
    per_token = 2 * (h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * i)
    attention = sum(2 * 2 * d * nq * tokens * (tokens + 1) // 2 for tokens in lengths)
    return layers * (per_token * sum(lengths) + attention) + len(lengths) * 2 * h * config["vocab_size"]


class L2Flush:
    """Writes a buffer larger than L2 (126 MB) so that the next timed kernel finds its inputs in HBM."""

    def __init__(self, torch):
        self.buffer = torch.empty(256 << 20, dtype=torch.uint8, device="cuda:0")

    def __call__(self):
        self.buffer.zero_()


def time_launches(torch, function, flush, repeats=20, warmup=3):
    """Median device time in microseconds of `function()`, its inputs flushed from L2 before every timed call."""
    for _ in range(warmup):
        function()
    times = []
    for _ in range(repeats):
        flush()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        function()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop) * 1e3)
    return round(statistics.median(times), 2)


def kernel_cases(torch, config, batch, context):
    """Inputs of the kernels that both arms time, at the sizes of a decode step of `batch` sequences at `context`
    positions and of a 2,048-token prefill."""
    generator = torch.Generator(device="cuda:0").manual_seed(0)
    h, i, d = config["hidden_size"], config["intermediate_size"], config["head_dim"]
    nq, nkv, vocab = config["num_attention_heads"], config["num_key_value_heads"], config["vocab_size"]
    bf16 = torch.bfloat16

    def randn(*shape, dtype=bf16):
        return torch.randn(*shape, generator=generator, device="cuda:0", dtype=torch.float32).to(dtype)

    return {
        "sizes": {"hidden": h, "intermediate": i, "head_dim": d, "heads": nq, "kv_heads": nkv, "vocab": vocab, "batch": batch, "context": context},
        "logits": randn(batch, vocab, dtype=torch.float32),
        "stacked_decode": randn(batch, 2 * i), "stacked_prefill": randn(2048, 2 * i),
        "hidden_decode": randn(batch, h), "branch_decode": randn(batch, h), "hidden_prefill": randn(2048, h), "branch_prefill": randn(2048, h),
        "norm_weight": (1 + 0.1 * randn(h, dtype=torch.float32)).to(bf16),
        "projected": randn(batch, (nq + 2 * nkv) * d), "head_weight": (1 + 0.1 * randn(d, dtype=torch.float32)).to(bf16),
        "history_k": randn(batch, nkv, context, d), "history_v": randn(batch, nkv, context, d),
    }


def reference_arm(args) -> int:
    why = ("taurs-ai/tau.rs is a Rust workspace whose dense Qwen3 model code lives in crates.io dependencies that are not on disk; no "
           "cargo/rustc is installed and there is no network, so there is no end-to-end reference number")
    record = {"impl": "reference", "unavailable": why}
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_kernels
        import torch

        if reference_kernels.available() and torch.cuda.is_available():
            record["kernels_us"] = reference_kernel_times(torch, reference_kernels, SHAPES[args.shape][0], args.batch or SHAPES[args.shape][1])
            record["kernels_note"] = ("the reference's generic kernels built unchanged (baseline/build_ref.py), timed alone with CUDA events, "
                                      "L2 flushed before each call; its kernels serve one sequence per launch, so a batch is that many launches")
    except Exception as error:   # the arm never fails: what could not be timed is said
        record["kernels_error"] = f"{type(error).__name__}: {error}"
    print(json.dumps(record))
    return 0


def reference_kernel_times(torch, ref, config, batch):
    context, capacity = 2048, SLOTS_PER_SEQUENCE
    case = kernel_cases(torch, config, batch, context)
    sizes = case["sizes"]
    nq, nkv, d = sizes["heads"], sizes["kv_heads"], sizes["head_dim"]
    flush = L2Flush(torch)
    bf16 = torch.bfloat16
    times = {}
    scratch = torch.empty(3 * (sizes["vocab"] // 1024 + 1), dtype=torch.int32, device="cuda:0")
    result = torch.empty(2, dtype=torch.int32, device="cuda:0")
    rows = [case["logits"][row].contiguous() for row in range(batch)]
    times[f"argmax_b{batch}"] = time_launches(torch, lambda: [ref.greedy_argmax(row, scratch, result) for row in rows], flush)
    for name in ("decode", "prefill"):
        stacked = case[f"stacked_{name}"]
        out = torch.empty(stacked.shape[0], stacked.shape[1] // 2, dtype=bf16, device="cuda:0")
        times[f"silu_mul_{name}"] = time_launches(torch, lambda: ref.silu_and_mul(stacked, out), flush)
        hidden, branch = case[f"hidden_{name}"], case[f"branch_{name}"]
        centered = (case["norm_weight"].float() - 1).to(bf16)
        normed, summed = torch.empty_like(hidden), torch.empty_like(hidden)
        times[f"rms_norm_{name}"] = time_launches(torch, lambda: ref.centered_rms_norm(hidden, centered, 1e-6, normed), flush)
        times[f"add_rms_norm_{name}"] = time_launches(torch, lambda: ref.fused_residual_rms_norm(hidden, branch, centered, summed, normed, 1e-6), flush)
    # One decoded token per sequence at position `context`: prepare, attention over tiles of 64 positions, merge.
    angles = torch.arange(capacity, dtype=torch.float32, device="cuda:0")[:, None] * torch.rand(d // 2, device="cuda:0")[None, :]
    cos, sin = torch.cos(angles).contiguous(), torch.sin(angles).contiguous()
    centered = (case["head_weight"].float() - 1).to(bf16)
    caches = []
    for index in range(batch):
        cache_k = torch.zeros(nkv, capacity, d, dtype=bf16, device="cuda:0")
        cache_v = torch.zeros(nkv, capacity, d, dtype=bf16, device="cuda:0")
        cache_k[:, :context] = case["history_k"][index]
        cache_v[:, :context] = case["history_v"][index]
        row = case["projected"][index]
        query_gate = torch.zeros(nq, 2 * d, dtype=bf16, device="cuda:0")
        query_gate[:, :d] = row[: nq * d].view(nq, d)
        caches.append((query_gate, row[nq * d : (nq + nkv) * d].view(nkv, d).contiguous(), row[(nq + nkv) * d :].view(nkv, d).contiguous(),
                       cache_k, cache_v))
    meta = torch.tensor([0, context], dtype=torch.int32, device="cuda:0")
    query = torch.empty(nq * d, dtype=bf16, device="cuda:0")
    out = torch.empty(nq * d, dtype=bf16, device="cuda:0")
    workspace = torch.empty(nq * (capacity // 64) * (d + 2), dtype=torch.float32, device="cuda:0")

    def decode_all():
        for query_gate, key, value, cache_k, cache_v in caches:
            ref.decode_attention_prepare(query_gate, key, value, centered, centered, cos, sin, query, cache_k, cache_v, meta, nq, nkv, d, capacity, d, 1e-6, context)
            ref.decode_attention(query, cache_k, cache_v, out, meta, workspace, nq, nkv, d, capacity, 64, context)

    times[f"decode_attention_b{batch}_ctx{context}"] = time_launches(torch, decode_all, flush)
    return times


def our_kernel_times(torch, kernels, config, batch):
    """This library's counterparts of `reference_kernel_times`, on the same inputs and with the same timing."""
    context = 2048
    case = kernel_cases(torch, config, batch, context)
    sizes = case["sizes"]
    nq, nkv, d = sizes["heads"], sizes["kv_heads"], sizes["head_dim"]
    flush = L2Flush(torch)
    bf16 = torch.bfloat16
    times = {}
    tokens = torch.empty(batch, dtype=torch.int32, device="cuda:0")
    valid = torch.empty(batch, dtype=torch.int32, device="cuda:0")
    times[f"argmax_b{batch}"] = time_launches(torch, lambda: kernels.argmax(case["logits"], tokens, valid), flush)
    weight = case["norm_weight"].float()
    for name in ("decode", "prefill"):
        stacked = case[f"stacked_{name}"]
        out = torch.empty(stacked.shape[0], stacked.shape[1] // 2, dtype=bf16, device="cuda:0")
        times[f"silu_mul_{name}"] = time_launches(torch, lambda: kernels.silu_mul(stacked, out), flush)
        hidden, branch = case[f"hidden_{name}"], case[f"branch_{name}"]
        normed, residual = torch.empty_like(hidden), hidden.clone()
        times[f"rms_norm_{name}"] = time_launches(torch, lambda: kernels.rms_norm(hidden, weight, 1e-6, normed), flush)
        times[f"add_rms_norm_{name}"] = time_launches(torch, lambda: kernels.add_rms_norm(branch, residual, weight, 1e-6, normed), flush)
    pages_per_sequence = SLOTS_PER_SEQUENCE // 64
    keys = torch.zeros(batch * pages_per_sequence, nkv, 64, d, dtype=bf16, device="cuda:0")
    values = torch.zeros_like(keys)
    for index in range(batch):
        first = index * pages_per_sequence
        keys[first : first + context // 64] = case["history_k"][index].view(nkv, context // 64, 64, d).transpose(0, 1)
        values[first : first + context // 64] = case["history_v"][index].view(nkv, context // 64, 64, d).transpose(0, 1)
    page_rows = torch.arange(batch * pages_per_sequence, dtype=torch.int32, device="cuda:0").view(batch, pages_per_sequence)
    seq_len = torch.full((batch,), context + 1, dtype=torch.int32, device="cuda:0")
    angles = torch.arange(SLOTS_PER_SEQUENCE, dtype=torch.float32, device="cuda:0")[:, None] * torch.rand(d // 2, device="cuda:0")[None, :]
    cos, sin = torch.cos(angles).contiguous(), torch.sin(angles).contiguous()
    out = torch.empty(batch, nq * d, dtype=bf16, device="cuda:0")
    head_weight = case["head_weight"].float()
    splits = kernels.decode_splits(batch, context + 1, nkv)
    times[f"decode_attention_b{batch}_ctx{context}"] = time_launches(torch, lambda: kernels.attention_decode(
        None, keys, values, out, seq_len, page_rows, nq, nkv, d, d ** -0.5, 0, splits,
        prepare=(case["projected"], head_weight, head_weight, 1e-6, cos, sin, d, True)), flush)
    return times


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=0, help="timed decode steps (0: the shape's default; 64 for the headline run)")
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes and workload (the headline run is 8b)")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers of the same sizes (named in the record)")
    parser.add_argument("--batch", type=int, default=0)
    parser.add_argument("--context", type=int, default=0, help="prompt length in tokens (the headline run uses 2,048)")
    parser.add_argument("--prefill-chunk", type=int, default=0, help="prompts enter the cache in chunks of this many tokens (0: the shape's default)")
    parser.add_argument("--skip-points", action="store_true", help="leave out the batch 1 and 64 points")
    parser.add_argument("--sections", default="prefill,decode,points,e2e",
                        help="which measurements to run: prefill, decode, points, e2e, kernels (the counterparts of the reference arm's kernels), "
                             "classes (time per kernel class of a decode step, outside a graph)")
    args = parser.parse_args()

    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU library")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3
    base_config, default_batch, default_context, default_steps, default_chunk = SHAPES[args.shape]
    full_layers = base_config["num_hidden_layers"]
    layers = args.layers or full_layers
    batch = args.batch or default_batch
    steps = args.steps or default_steps
    unequal = default_context == 0 and not args.context
    prompt_tokens = args.context or default_context
    headline = args.shape == "8b" and (batch, prompt_tokens) == (8, 2048)

    import numpy as np
    import torch

    import tau_rs_b200
    from tau_rs_b200 import Engine, StepEntry
    from tau_rs_b200.csrc import kernels

    torch.cuda.set_device(0)
    peaks = measured_peaks()
    config = dict(base_config, num_hidden_layers=layers)
    vocab = config["vocab_size"]
    rng = np.random.default_rng(3 if unequal else 0)
    lengths = rng.integers(1, 1025, size=batch).tolist() if unequal else [prompt_tokens] * batch
    longest = max(lengths)
    slots_per_sequence = max(SLOTS_PER_SEQUENCE, (longest + steps + 64 + 63) // 64 * 64)
    chunk = args.prefill_chunk or default_chunk or sum(lengths)
    sections = set(args.sections.split(","))
    if args.skip_points or not headline:
        sections.discard("points")

    model = tau_rs_b200.random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
    weight_bytes = model.weight_bytes()

    def prompts(counts):
        return [rng.integers(0, vocab, size=count).tolist() for count in counts]

    def fresh_engine(count):
        return Engine(model, max_tokens=count * slots_per_sequence, max_sequence_tokens=slots_per_sequence)

    def timed(function):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        function()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop)

    def feed_prompts(engine, slots, texts, want_last):
        """The prompts packed along one token axis, in chunks of at most `chunk` tokens over the batch."""
        fed = [0] * len(texts)
        while any(done < len(text) for done, text in zip(fed, texts)):
            budget, entries = chunk, []
            for index, (slot, text) in enumerate(zip(slots, texts)):
                count = min(len(text) - fed[index], budget)
                if count <= 0:
                    continue
                ends = fed[index] + count == len(text)
                entries.append(StepEntry(slot, text[fed[index] : fed[index] + count], [count - 1] if ends and want_last else []))
                fed[index] += count
                budget -= count
            engine.step(entries)

    # ---- prefill: one prompt of the headline length, or the workload's whole batch of prompts -----------------------
    prefill = None
    if "prefill" in sections:
        prefill_lengths = [prompt_tokens] if headline or not unequal and args.shape == "8b" else lengths
        engine = fresh_engine(len(prefill_lengths))
        texts = prompts(prefill_lengths)

        def one_prefill():
            slots = [engine.open_sequence() for _ in texts]
            feed_prompts(engine, slots, texts, True)
            for slot in slots:
                engine.close_sequence(slot)

        for _ in range(3 if sum(prefill_lengths) <= 8192 else 1):
            one_prefill()
        prefill_ms = min(timed(one_prefill) for _ in range(3 if sum(prefill_lengths) <= 8192 else 1))
        flops = prefill_flops(config, layers, prefill_lengths)
        total = sum(prefill_lengths)
        prefill = {"value": round(total / prefill_ms * 1e3, 1), "tokens": total, "ms": round(prefill_ms, 3),
                   "frac": round(flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4), "of": peaks["source"]}
        del engine
        torch.cuda.empty_cache()

    # ---- decode -----------------------------------------------------------------------------
    def decode_run(count, run_lengths, run_steps, warmup, sample_clocks=False, classes=False):
        """Device time of `run_steps` decode steps of `count` sequences that hold prompts of the given lengths."""
        engine = fresh_engine(count)
        slots = [engine.open_sequence() for _ in range(count)]
        feed_prompts(engine, slots, prompts(run_lengths), False)
        feed = rng.integers(0, vocab, size=(warmup + run_steps, count)).tolist()
        chosen = torch.empty((2, count), dtype=torch.int32, device="cuda:0")
        if classes:
            engine.use_graphs = False

        def one_step(index):
            logits = engine.step([StepEntry(slot, [feed[index][row]], [0]) for row, slot in enumerate(slots)])
            kernels.argmax(logits, chosen[0], chosen[1])

        for index in range(warmup):
            one_step(index)
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.start()
        # The prompts' prefill ran at the power cap and leaves the SM clock low for some dozens of steps; every decode
        # timing waits the same 0.3 s before its timed steps, so that all of them are taken at the clocks of decoding.
        torch.cuda.synchronize()
        time.sleep(0.3)
        before = kernels.launch_count()
        per_class = None
        if classes:
            torch.cuda.synchronize()
            kernels.start_timing()
        elapsed = timed(lambda: [one_step(warmup + index) for index in range(run_steps)])
        if classes:
            per_class = {name: round(value / run_steps, 4) for name, value in kernels.take_timing(stop=True).items()}
        launches = kernels.launch_count() - before
        record = clocks.stop() if clocks else None
        live_bytes = engine.cache.live_bytes()
        layout_ints = engine.last_step_ints
        for slot in slots:
            engine.close_sequence(slot)
        del engine
        torch.cuda.empty_cache()
        return elapsed, launches, record, live_bytes, layout_ints, per_class

    value = ms_per_step = launches = clocks = roofline = None
    live_bytes = layout_ints = 0
    if "decode" in sections:
        elapsed, launches, clocks, live_bytes, layout_ints, _ = decode_run(batch, lengths, steps, args.warmup, sample_clocks=True)
        ms_per_step = round(elapsed / steps, 4)
        value = round(batch * steps / (elapsed * 1e-3), 1)
        achieved = (weight_bytes + live_bytes) / (elapsed / steps * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks["source"]}

    points = {}
    if "points" in sections:
        for count, point_steps in ((1, max(16, steps // 2)), (64, max(16, steps // 2))):
            point_elapsed = decode_run(count, [prompt_tokens] * count, point_steps, 3)[0]
            points[f"decode_b{count}"] = round(count * point_steps / (point_elapsed * 1e-3), 1)

    extra = {}
    if "classes" in sections:
        class_steps = min(steps, 16)
        extra["ms_per_step_by_kernel_class"] = decode_run(batch, lengths, class_steps, 3, classes=True)[5]
    if "kernels" in sections:
        extra["kernels_us"] = our_kernel_times(torch, kernels, config, batch)

    # ---- end to end through generate(): host tokens in, host tokens out, every step ---------------
    e2e = None
    if "e2e" in sections:
        engine = fresh_engine(batch)
        batch_prompts = prompts(lengths)
        generate_chunk = chunk if chunk < sum(lengths) else None
        # One call: the prompts, then `warmup` untimed decode steps and `steps` timed ones.  The metrics' sink sees the counters at
        # every token boundary; the rate is decoded tokens over decode time between step `warmup` and step `warmup + steps`.
        def end_to_end(**sampling):
            marks = []
            watched = tau_rs_b200.GenerationMetrics(log_interval_s=0.0, sink=lambda record: marks.append((record["decode_steps"], record["decode_tokens"], record["decode_ms"])))
            output = tau_rs_b200.generate(engine, batch_prompts, max_new_tokens=args.warmup + steps + 1, stop_tokens=(),
                                          prefill_chunk_tokens=generate_chunk, metrics=watched, **sampling)
            marks.append((output.metrics.decode_steps, output.metrics.decode_tokens, output.metrics.decode_ms))
            first = max((mark for mark in marks if mark[0] <= args.warmup), default=(0, 0, 0.0))
            last = marks[-1]
            return (last[1] - first[1]) / ((last[2] - first[2]) * 1e-3), round((last[1] - first[1]) / batch)

        tau_rs_b200.generate(engine, batch_prompts, max_new_tokens=3, stop_tokens=(), prefill_chunk_tokens=generate_chunk)   # graphs captured, pools sized
        rate, timed_steps = end_to_end()
        e2e = {"value": round(rate, 1), "unit": "tok/s", "h2d_bytes_per_step": layout_ints * 4, "d2h_bytes_per_step": 2 * batch * 4,
               "steps": timed_steps}
        if unequal:   # the workload's second half: temperature 0.8
            e2e["temperature_0.8_value"] = round(end_to_end(temperature=0.8, seed=3)[0], 1)
        del engine

    names = {"8b": "Qwen3-8B", "0.6b": "Qwen3-0.6B", "32b": "Qwen3-32B"}
    what = f"{prompt_tokens:,}-token prompts" if not unequal else "prompts of 1 to 1,024 tokens (uniform, seed 3)"
    record = {
        "metric": f"decode tok/s at batch {batch}, {what} ({names[args.shape]} bf16)", "value": value, "unit": "tok/s", "n_gpus": 1,
        "steps": steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: uniform random token ids, random-init weights N(0, 0.02)", "impl": "ours",
        "config": {
            "model": f"{names[args.shape]} shape", "layers": layers, "layers_full": full_layers, "hidden": config["hidden_size"],
            "heads": config["num_attention_heads"], "kv_heads": config["num_key_value_heads"], "head_dim": config["head_dim"],
            "intermediate": config["intermediate_size"], "vocab": vocab, "global_batch": batch,
            "seq_len": prompt_tokens if not unequal else round(sum(lengths) / batch),
            "cache_slots_per_seq": slots_per_sequence, "rope_theta": config["rope_theta"], "rms_norm_eps": config["rms_norm_eps"],
            "tied": config["tie_word_embeddings"], "parallelism": "single GPU", "l2": "inputs (the weights) exceed L2; no flush",
            "weight_bytes": weight_bytes, "kv_bytes_per_step": live_bytes,
        },
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points, **extra,
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
