"""Decode and prefill throughput of the Qwen3-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  `value` is decoded tokens per second at batch 8 with 2,048-token
prompts (a step is one decode step of the whole batch), timed on the device with CUDA events
around exactly K steps; `e2e` is the same through `tau_rs_b200.generate` with host tokens in
and out of every step; `prefill` is one 2,048-token prompt; `points` are batch 1 and 64.
The weights (15 GB) are far larger than L2, so nothing is flushed between iterations.
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

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "attention_bias": False,
    "max_position_embeddings": 40960, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
FULL_LAYERS = 36
PROMPT_TOKENS = 2048
SLOTS_PER_SEQUENCE = 8192
METRIC = "decode tok/s at batch 8, 2,048-token prompts (Qwen3-8B bf16)"


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


def prefill_flops(config, layers, tokens):
    h, i, d = config["hidden_size"], config["intermediate_size"], config["head_dim"]
    nq, nkv = config["num_attention_heads"], config["num_key_value_heads"]
    per_token = 2 * (h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * i)
    attention = 2 * 2 * d * nq * tokens * (tokens + 1) // 2      # q.k and p.v over the causal half
    return layers * (per_token * tokens + attention) + 2 * h * config["vocab_size"]


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers of the same sizes (named in the record)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=PROMPT_TOKENS, help="prompt length in tokens (the headline run uses 2,048)")
    parser.add_argument("--prefill-chunk", type=int, default=0, help="prompts enter the cache in chunks of this many tokens (0: whole)")
    parser.add_argument("--skip-points", action="store_true", help="leave out the batch 1 and 64 points")
    parser.add_argument("--sections", default="prefill,decode,points,e2e", help="which measurements to run (for profiling a part alone)")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "tau.rs is a Rust workspace whose Qwen3 model code lives in crates.io "
                          "dependencies that are not on disk; no cargo/rustc is installed and there is no network"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU library")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    prompt_tokens = args.context
    slots_per_sequence = max(SLOTS_PER_SEQUENCE, (prompt_tokens + 1024 + 63) // 64 * 64)
    chunk = args.prefill_chunk if args.prefill_chunk > 0 else prompt_tokens

    import numpy as np
    import torch

    import tau_rs_b200
    from tau_rs_b200 import Engine, StepEntry
    from tau_rs_b200.csrc import kernels

    torch.cuda.set_device(0)
    peaks = measured_peaks()
    config = dict(QWEN3_8B, num_hidden_layers=args.layers)
    model = tau_rs_b200.random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
    weight_bytes = model.weight_bytes()
    rng = np.random.default_rng(0)
    vocab = config["vocab_size"]

    def prompts(count):
        return [rng.integers(0, vocab, size=prompt_tokens).tolist() for _ in range(count)]

    def fresh_engine(batch):
        return Engine(model, max_tokens=batch * slots_per_sequence, max_sequence_tokens=slots_per_sequence)

    def timed(function):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        function()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop)

    sections = set(args.sections.split(","))
    if args.skip_points:
        sections.discard("points")

    # ---- prefill of one 2,048-token prompt ------------------------------------------------
    engine = fresh_engine(1)
    (prompt,) = prompts(1)

    def one_prefill():
        slot = engine.open_sequence()
        for start in range(0, prompt_tokens, chunk):
            piece = prompt[start : start + chunk]
            engine.step([StepEntry(slot, piece, [len(piece) - 1] if start + chunk >= prompt_tokens else [])])
        engine.close_sequence(slot)

    prefill = None
    if "prefill" in sections:
        for _ in range(3):
            one_prefill()
        prefill_ms = min(timed(one_prefill) for _ in range(3))
        flops = prefill_flops(config, args.layers, prompt_tokens)
        prefill = {"value": round(prompt_tokens / prefill_ms * 1e3, 1), "tokens": prompt_tokens, "ms": round(prefill_ms, 3),
                   "frac": round(flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4), "of": peaks["source"]}
    del engine

    # ---- decode -----------------------------------------------------------------------------
    def decode_run(batch, steps, warmup, sample_clocks=False):
        """Device time of `steps` decode steps of `batch` sequences that hold prompts of the chosen length."""
        engine = fresh_engine(batch)
        slots = [engine.open_sequence() for _ in range(batch)]
        for slot, tokens in zip(slots, prompts(batch)):      # prompts one by one: bounded activations
            for start in range(0, prompt_tokens, chunk):
                engine.step([StepEntry(slot, tokens[start : start + chunk], [])])
        feed = rng.integers(0, vocab, size=(warmup + steps, batch)).tolist()
        sampler = tau_rs_b200.Sampler()
        chosen = torch.empty((2, batch), dtype=torch.int32, device="cuda:0")

        def one_step(index):
            logits = engine.step([StepEntry(slot, [feed[index][row]], [0]) for row, slot in enumerate(slots)])
            kernels.argmax(logits, chosen[0], chosen[1])

        for index in range(warmup):
            one_step(index)
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.start()
            time.sleep(0.3)
        before = kernels.launch_count()
        elapsed = timed(lambda: [one_step(warmup + index) for index in range(steps)])
        launches = kernels.launch_count() - before
        record = clocks.stop() if clocks else None
        live_bytes = engine.cache.live_bytes()
        layout_ints = engine.last_step_ints
        for slot in slots:
            engine.close_sequence(slot)
        del engine
        torch.cuda.empty_cache()
        return elapsed, launches, record, live_bytes, layout_ints

    value = ms_per_step = launches = clocks = roofline = None
    live_bytes = layout_ints = 0
    if "decode" in sections:
        elapsed, launches, clocks, live_bytes, layout_ints = decode_run(args.batch, args.steps, args.warmup, sample_clocks=True)
        ms_per_step = round(elapsed / args.steps, 4)
        value = round(args.batch * args.steps / (elapsed * 1e-3), 1)
        achieved = (weight_bytes + live_bytes) / (elapsed / args.steps * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks["source"]}

    points = {}
    if "points" in sections:
        for batch, steps in ((1, max(16, args.steps // 2)), (64, max(16, args.steps // 2))):
            point_elapsed, _, _, _, _ = decode_run(batch, steps, 3)
            points[f"decode_b{batch}"] = round(batch * steps / (point_elapsed * 1e-3), 1)

    # ---- end to end through generate(): host tokens in, host tokens out, every step ---------------
    e2e = None
    if "e2e" in sections:
        engine = fresh_engine(args.batch)
        batch_prompts = prompts(args.batch)
        tau_rs_b200.generate(engine, batch_prompts, max_new_tokens=args.warmup + 1, stop_tokens=(), prefill_chunk_tokens=chunk)
        output = tau_rs_b200.generate(engine, batch_prompts, max_new_tokens=args.steps + 1, stop_tokens=(), prefill_chunk_tokens=chunk)
        e2e = {"value": round(output.metrics.decode_tokens_per_second, 1), "unit": "tok/s",
               "h2d_bytes_per_step": layout_ints * 4, "d2h_bytes_per_step": 2 * args.batch * 4,
               "steps": output.metrics.decode_steps}

    record = {
        "metric": METRIC if (args.batch, prompt_tokens) == (8, PROMPT_TOKENS) else f"decode tok/s at batch {args.batch}, {prompt_tokens:,}-token prompts (Qwen3-8B bf16)", "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, random-init weights N(0, 0.02)", "impl": "ours",
        "config": {
            "model": "Qwen3-8B shape", "layers": args.layers, "layers_full": FULL_LAYERS, "hidden": config["hidden_size"],
            "heads": config["num_attention_heads"], "kv_heads": config["num_key_value_heads"], "head_dim": config["head_dim"],
            "intermediate": config["intermediate_size"], "vocab": vocab, "global_batch": args.batch, "seq_len": prompt_tokens,
            "cache_slots_per_seq": slots_per_sequence, "rope_theta": config["rope_theta"], "rms_norm_eps": config["rms_norm_eps"],
            "tied": False, "parallelism": "single GPU", "l2": "inputs (15 GB of weights) exceed L2; no flush",
            "weight_bytes": weight_bytes, "kv_bytes_per_step": live_bytes,
        },
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points,
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
