"""Writes tests/golden/plain_tiny.json from the plain implementation (CPU, float32).

tau.rs's dense Qwen3 layer math is not in its tree (crates/models/src/qwen3.rs:8-10 re-exports
an external crate) and no Rust toolchain is installed, so the reference's own model code cannot
be run here; these values therefore pin the plain implementation, which rests on the formulas,
against accidental change.  The shape of the record follows the reference's own numerics
fixtures (crates/models/src/qwen3_5.rs:91-166: a slice of logits, the argmax, a tolerance of
2e-5 absolute).  Run: python tests/golden/make_plain_golden.py
"""
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import numpy as np  # noqa: E402

import plain_model  # noqa: E402
import tiny_configs  # noqa: E402

record = {}
with tempfile.TemporaryDirectory() as root:
    for which in ("A", "B"):
        folder = tiny_configs.write_tiny(root, which)
        config = plain_model.read_plain_config(folder)
        weights = plain_model.read_plain_weights(folder)
        tokens = np.random.default_rng(100).integers(0, config.vocab_size, size=21).tolist()
        logits = plain_model.forward_logits(config, weights, tokens)
        record[which] = {
            "tokens": tokens,
            "last_logits_first_16": [float(value) for value in logits[-1, :16]],
            "last_argmax": int(logits[-1].argmax()),
            "greedy_6": plain_model.greedy_generate(config, weights, tokens, 6),
        }
with open(os.path.join(HERE, "plain_tiny.json"), "w") as handle:
    json.dump(record, handle, indent=1)
print("wrote plain_tiny.json")
