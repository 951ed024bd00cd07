"""Trace replay: feeds given token ids through a model step by step and writes logits.

Nothing is sampled.  The model, cache and step function are the library's own
(`load_engine`, `Engine.step`); this module only translates the line protocol.  Each input
line is a JSON object `{"step": k, "entries": [{"id", "tokens", "want"}], "end": [ids]}`; for a
step that wants something the logits at the wanted places are written to `<out>/<k>.f32` as
little-endian 32-bit floats `[wanted, vocab]`, in the order of the entries and of `want`;
after every step `done <k>` is printed and flushed.  The reference has only an outbound
trace of this kind of record (crates/metrics/src/trace.rs:88-106).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import numpy as np


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32", "bf16", "f32"],
                        help="bfloat16: the kernels and precisions that serving uses; float32: everything in true 32-bit")
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time (each rounded up to 64); sizes the cache")
    return parser


def run(arguments, lines=None, out=None) -> int:
    lines = sys.stdin if lines is None else lines
    out = sys.stdout if out is None else out
    print(f"[trace_run] loading {arguments.model} ({arguments.dtype})", file=sys.stderr, flush=True)
    from .api import load_engine
    from .engine.batch import StepEntry

    engine = load_engine(arguments.model, arguments.dtype, "gpu", max_tokens=arguments.max_tokens,
                         enforce_declared_dtype=False)
    os.makedirs(arguments.out, exist_ok=True)
    slots: Dict[str, int] = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            key = str(item["id"])
            if key not in slots:
                slots[key] = engine.open_sequence()
            entries.append(StepEntry(slots[key], [int(token) for token in item["tokens"]], [int(place) for place in item.get("want", [])]))
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                values = logits.float().cpu().numpy().astype("<f4", copy=False)
                with open(os.path.join(arguments.out, f"{step}.f32"), "wb") as handle:
                    handle.write(np.ascontiguousarray(values).tobytes())
        for key in record.get("end", []):
            slot = slots.pop(str(key), None)
            if slot is not None:
                engine.close_sequence(slot)
        print(f"done {step}", file=out, flush=True)
    return 0


def main(argv=None) -> int:
    return run(build_parser().parse_args(argv))
