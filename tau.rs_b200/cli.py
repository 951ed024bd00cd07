"""Command line in the manner of `tau-server` (crates/server/src/args.rs:346-446), for token ids instead of chat text.

Options that the reference has keep its names and meanings: `-m/--model PATH`,
`--device auto|gpu|cpu` (args.rs: auto is CUDA GPU 0; this library has no CPU path, so `cpu`
is refused as the reference refuses bfloat16 there), `--dtype auto|f32|bf16` (auto: bf16 if
the folder declares it), `--optimize-kernel true|false` (false: this library's plain kernels, as the
reference's are Candle's), `--cuda-graph none|full`, `--attention-block-size 32|64|128|256` (context tokens per block of decode attention; the
reference's default is a fixed size, here the number of blocks follows the batch and the context unless it is given), `--prefill-chunk-size N`, `--metrics`
(an `inference_metrics {...}` line on stderr, crates/metrics/src/serving.rs:35-54),
`--vram-metrics` (an `inference_vram_metrics {...}` line on stderr, crates/metrics/src/memory.rs:119-138),
`--tracing` (an `inference_trace {...}` line on stdout with prompt ids, generated ids and
per-step logit checksums, crates/metrics/src/trace.rs:22-52,88-106; logits then go to the
host and the host selector of crates/engine/src/generation.rs:81-95 is not needed because
the device selector has the same semantics), and `--max-tokens N` as the output limit of a
request (the request field `max_tokens`, crates/server/src/chat_completions_handler/
request.rs:27-110; default: the folder's generation settings, else 16).  The server, chat
template and MoE options have no counterpart here.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
import time
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="tau", description="Generate token ids with a local safetensors model on one B200.")
    model = parser.add_argument_group("Model options")
    model.add_argument("-m", "--model", metavar="PATH", help="Local safetensors model directory.")
    model.add_argument("--device", default="auto", choices=["auto", "gpu", "cpu"], help="Execution device. [default: auto] auto/gpu: CUDA GPU 0; cpu is not available.")
    model.add_argument("--dtype", default="auto", choices=["auto", "f32", "bf16", "float32", "bfloat16"],
                       help="Model precision. [default: auto] auto: BF16 if the folder declares it, else F32. F32 is true 32-bit throughout.")
    model.add_argument("--random-weights", metavar="CONFIG_JSON", help="Write a model folder with random weights for this config.json to --model and exit unless prompts are given.")
    model.add_argument("--seed", type=int, default=0, help="Seed of random weights and of temperature sampling. [default: 0]")
    model.add_argument("--norm-jitter", type=float, default=0.0, help="Random weights: norm weights are 1 + N(0, jitter). [default: 0]")
    execution = parser.add_argument_group("Execution options")
    execution.add_argument("--optimize-kernel", default="true", choices=["true", "false"],
                           help="Prefer optimized kernels. [default: true] false: the plain kernels that the others are checked against.")
    execution.add_argument("--cuda-graph", default="full", choices=["none", "full"], help="CUDA graph policy for decode steps. [default: full]")
    execution.add_argument("--attention-block-size", type=int, default=None, choices=[32, 64, 128, 256], metavar="32|64|128|256",
                           help="Context tokens per block of decode attention. [default: chosen from the batch and the context]")
    execution.add_argument("--prefill-chunk-size", type=int, default=8192, metavar="N", help="Most prompt tokens per prefill step, over the whole batch. [default: 8192]")
    execution.add_argument("--max-batch", type=int, default=64, metavar="N", help="Most requests that start together. [default: 64]")
    execution.add_argument("--cache-tokens", type=int, default=None, metavar="N", help="Tokens the cache holds (each live request rounded up to 64). [default: what the requests need]")
    request = parser.add_argument_group("Request options")
    request.add_argument("--prompt-ids", action="append", default=[], metavar="1,2,3", help="Token ids of one prompt; may be given several times.")
    request.add_argument("--prompt-file", metavar="PATH", help="File of prompts: a JSON list of lists of token ids, or one prompt a line (ids parted by commas or spaces).")
    request.add_argument("--max-tokens", type=int, default=None, metavar="N", help="Most tokens to generate per request. [default: generation settings of the folder, else 16]")
    request.add_argument("--temperature", type=float, default=0.0, help="0: greedy. [default: 0]")
    request.add_argument("--stop-ids", default=None, metavar="1,2", help="Stop token ids. [default: eos_token_id of the folder]")
    logging = parser.add_argument_group("Logging options")
    logging.add_argument("--metrics", action="store_true", help="Log live decode t/s to stderr. [default: off] Every ~5s during generation and at completion.")
    logging.add_argument("--tracing", action="store_true", help="Log numerical traces (token ids, logit checksums) to stdout. [default: off]")
    logging.add_argument("--hbm-gbs", type=float, default=None, metavar="GB/s",
                         help="The device's measured copy bandwidth; with --metrics the report then carries the decode steps' fraction of that roofline.")
    logging.add_argument("--vram-metrics", action="store_true", help="Sample process VRAM; log peak to stderr. [default: off] Independent of --metrics and --tracing.")
    return parser


def _ids(text: str) -> List[int]:
    return [int(part) for part in text.replace(",", " ").split()]


def read_prompt_file(path: str) -> List[List[int]]:
    """A JSON list of prompts (each a list of token ids), or one prompt a line with ids parted by commas or spaces."""
    with open(path) as handle:
        text = handle.read()
    try:
        if text.lstrip().startswith("["):
            prompts = json.loads(text)
            if isinstance(prompts, list) and all(isinstance(prompt, list) and prompt and all(isinstance(token, int) and not isinstance(token, bool) for token in prompt) for prompt in prompts):
                return prompts
            raise ValueError("not a list of non-empty lists of integers")
        return [_ids(line) for line in text.splitlines() if line.strip()]
    except ValueError as error:
        raise SystemExit(f"--prompt-file {path}: expected a JSON list of lists of token ids, or one prompt of ids a line ({error})")


def logit_snapshot(values, token: int) -> dict:
    """What the reference's trace keeps of one vector of logits (crates/metrics/src/logits.rs:10-60): the count, how many
    are finite, the SHA-256 of all of them as little-endian 32-bit floats, up to 16 samples spread evenly over the
    vocabulary (`token_id = i * (count - 1) / (samples - 1)`; a value that is not finite is null) and the chosen logit."""
    import numpy as np

    values = np.ascontiguousarray(values, dtype="<f4")
    count = int(values.size)
    finite = np.isfinite(values)
    sample_count = min(count, 16)
    samples = []
    for i in range(sample_count):
        token_id = i * max(count - 1, 0) // max(sample_count - 1, 1)
        samples.append({"token_id": token_id, "value": float(values[token_id]) if finite[token_id] else None})
    selected = float(values[token]) if 0 <= token < count and finite[token] else None
    return {"count": count, "finite_count": int(finite.sum()), "sha256_f32_le": hashlib.sha256(values.tobytes()).hexdigest(),
            "samples": samples, "selected_logit": selected}


class _Tracer:
    """Wraps a selector: copies each step's logits to the host and records what the reference's trace records for a
    step (crates/metrics/src/trace.rs:88-106): its phase, the cache offset it ran at (0 for the prompt, then
    `prompt + tokens so far - 1`, crates/engine/src/model_engine/generation.rs:181-183), how many tokens it brought,
    the chosen token, whether that is a stop token, when it started and how long it took, and the logits' snapshot."""

    def __init__(self, select, prompts, stop):
        self.select, self.steps, self.started = select, [], time.perf_counter()
        self.prompts, self.stop = prompts, frozenset(stop)
        self.boundary = self.started

    def __call__(self, logits, request_ids, token_indices):
        begin = self.boundary
        tokens = self.select(logits, request_ids, token_indices)
        host = logits.float().cpu().numpy()
        end = time.perf_counter()
        from .csrc import kernels

        by_class = kernels.take_timing()      # milliseconds per kernel class since the select before (empty unless timing is on)
        for row, (request, index, token) in enumerate(zip(request_ids, token_indices, tokens)):
            prompt_tokens = len(self.prompts[request])
            self.steps.append({
                "index": len(self.steps), "request": request, "phase": "prefill" if index == 0 else "decode", "token_index": index,
                "cache_offset": 0 if index == 0 else prompt_tokens + index - 1, "input_tokens": prompt_tokens if index == 0 else 1,
                "token_id": int(token), "is_eos": int(token) in self.stop,
                "start_us": round((begin - self.started) * 1e6, 1), "duration_us": round((end - begin) * 1e6, 1),
                "logits": logit_snapshot(host[row], int(token)),
                **({"kernel_class_ms": by_class} if by_class and row == 0 else {}),
            })
        self.boundary = time.perf_counter()
        return tokens


def main(argv: Optional[List[str]] = None) -> int:
    parser = build_parser()
    args = parser.parse_args(argv)
    if args.model is None:
        parser.error("--model is required")
    if args.prefill_chunk_size <= 0:
        parser.error("--prefill-chunk-size must be positive")
    if args.random_weights:
        from .weights import write_random_model

        with open(args.random_weights) as handle:
            config = json.load(handle)
        storage = "float32" if args.dtype in ("f32", "float32") else "bfloat16"
        write_random_model(args.model, config, seed=args.seed, norm_jitter=args.norm_jitter, storage=storage)
        print(f"wrote {args.model} (seed {args.seed}, {storage})", file=sys.stderr)
    prompts = [_ids(text) for text in args.prompt_ids]
    if args.prompt_file:
        prompts += read_prompt_file(args.prompt_file)
    if not prompts:
        if args.random_weights:
            return 0
        parser.error("give --prompt-ids or --prompt-file")

    from .api import load_model
    from .config.generation import GenerationConfig
    from .engine.generate import GenerationMetrics, generate_tokens
    from .engine.step import Engine
    from .sampling.sampler import Sampler, SamplingParams

    from .csrc import kernels

    kernels.prefer_optimized(args.optimize_kernel == "true")
    model = load_model(args.model, args.dtype, args.device)
    settings: GenerationConfig = model.generation_config
    limit = args.max_tokens if args.max_tokens is not None else settings.max_new_tokens
    stop = _ids(args.stop_ids) if args.stop_ids is not None else settings.eos_token_ids
    cache_tokens = args.cache_tokens
    if cache_tokens is None:
        needs = sorted((-(-(len(prompt) + limit) // 64) * 64 for prompt in prompts), reverse=True)
        cache_tokens = max(64, sum(needs[: args.max_batch]))
    engine = Engine(model, cache_tokens)
    engine.use_graphs = engine.use_graphs and args.cuda_graph == "full"
    engine.attention_block_size = args.attention_block_size
    select = Sampler(SamplingParams(args.temperature, args.seed))   # the object, not its method: the loop then decodes one step ahead
    tracer = _Tracer(select, prompts, stop) if args.tracing else None
    if tracer:
        # A traced run times the kernel classes of every step with CUDA events (crates/metrics/src/timing.rs:83-183 does so
        # for its decode phases), which needs the launches themselves: no replayed graph.
        engine.use_graphs = False
        kernels.start_timing()
    metrics = GenerationMetrics(peak_gb_per_second=args.hbm_gbs)
    if args.metrics:   # live: every ~5 s during generation and at completion
        metrics.log_interval_s = 5.0
        metrics.sink = lambda record: print("inference_metrics " + json.dumps(record), file=sys.stderr, flush=True)
    memory = None
    if args.vram_metrics:
        from . import vram

        memory = vram.device_sampler().start()
    started = time.perf_counter()
    try:
        results = generate_tokens(engine, prompts, limit, tracer or select, stop, args.max_batch, args.prefill_chunk_size, metrics)
    except Exception as error:
        if memory is not None:
            vram.report(memory.finish(), args.model, error=str(error))
        if args.metrics:
            metrics.sink(dict(metrics.report("error"), error=str(error)))
        raise
    elapsed = time.perf_counter() - started
    if memory is not None:
        vram.report(memory.finish(), args.model)
    for index, result in enumerate(results):
        print(json.dumps({"request": index, "prompt_tokens": result.prompt_tokens, "completion_tokens": len(result.tokens),
                          "tokens": result.tokens, "finish_reason": result.finish_reason}))
    if tracer:
        print("inference_trace " + json.dumps({
            "schema": "tau_rs_b200/1", "prompts": prompts, "generated": [result.tokens for result in results], "steps": tracer.steps,
            "summary": {"decode_tokens_per_second": metrics.decode_tokens_per_second, "elapsed_ms": elapsed * 1e3}}))
    if args.metrics:
        metrics.sink(metrics.report("ok"))
    return 0
