"""The command line's own decisions, without a GPU: options, the random-weights mode, refusals."""
import json
import os

import pytest

import tiny_configs
from tau_rs_b200 import cli


def test_options_keep_the_reference_names():
    """crates/server/src/args.rs:346-446: the names and values of the options that this library has a meaning for."""
    parser = cli.build_parser()
    args = parser.parse_args(["-m", "folder", "--device", "gpu", "--dtype", "bf16", "--optimize-kernel", "false", "--cuda-graph", "none",
                              "--attention-block-size", "128", "--prefill-chunk-size", "256", "--metrics", "--tracing", "--vram-metrics",
                              "--prompt-ids", "1,2,3", "--prompt-ids", "4 5", "--max-tokens", "7"])
    assert (args.model, args.device, args.dtype, args.optimize_kernel, args.cuda_graph) == ("folder", "gpu", "bf16", "false", "none")
    assert (args.attention_block_size, args.prefill_chunk_size, args.max_tokens) == (128, 256, 7)
    assert args.metrics and args.tracing and args.vram_metrics and args.prompt_ids == ["1,2,3", "4 5"]
    defaults = parser.parse_args(["--model", "folder"])
    assert (defaults.device, defaults.dtype, defaults.optimize_kernel, defaults.cuda_graph) == ("auto", "auto", "true", "full")
    assert defaults.attention_block_size is None and not (defaults.metrics or defaults.tracing or defaults.vram_metrics)
    for bad in (["--attention-block-size", "48"], ["--cuda-graph", "sometimes"], ["--optimize-kernel", "maybe"], ["--device", "tpu"]):
        with pytest.raises(SystemExit):
            parser.parse_args(["--model", "folder"] + bad)


def test_random_weights_mode_writes_a_folder_and_stops(tmp_path, capsys):
    config = tmp_path / "config.json"
    config.write_text(json.dumps(tiny_configs.CONFIGS["A"]))
    folder = tmp_path / "model"
    assert cli.main(["--model", str(folder), "--random-weights", str(config), "--seed", "4", "--dtype", "f32"]) == 0
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    written = json.loads((folder / "config.json").read_text())
    assert written["architectures"] == ["Qwen3ForCausalLM"] and written["hidden_size"] == tiny_configs.CONFIGS["A"]["hidden_size"]
    assert "seed 4" in capsys.readouterr().err


def test_refusals_are_said_before_anything_is_loaded(tmp_path):
    with pytest.raises(SystemExit):
        cli.main([])                                                   # no --model
    with pytest.raises(SystemExit):
        cli.main(["--model", str(tmp_path)])                           # no prompts
    with pytest.raises(SystemExit):
        cli.main(["--model", str(tmp_path), "--prompt-ids", "1", "--prefill-chunk-size", "0"])
    folder = tiny_configs.write_tiny(str(tmp_path), "A")
    with pytest.raises(Exception, match="cpu is not available"):      # the reference runs F32 there; this library has no CPU path
        cli.main(["--model", folder, "--prompt-ids", "1,2", "--device", "cpu"])


def test_the_trace_snapshot_of_a_vector_of_logits():
    """crates/metrics/src/logits.rs:10-60: hash over every value as little-endian 32-bit floats, 16 samples spread over
    the vocabulary (first and last included), null for values that are not finite."""
    import hashlib

    import numpy as np

    values = np.arange(100, dtype=np.float32) * 0.5
    values[33] = np.inf
    values[99] = np.nan
    snapshot = cli.logit_snapshot(values, 98)
    assert snapshot["count"] == 100 and snapshot["finite_count"] == 98 and snapshot["selected_logit"] == 49.0
    assert snapshot["sha256_f32_le"] == hashlib.sha256(values.astype("<f4").tobytes()).hexdigest()
    assert [sample["token_id"] for sample in snapshot["samples"]] == [i * 99 // 15 for i in range(16)]
    assert snapshot["samples"][0]["value"] == 0.0 and snapshot["samples"][5]["value"] is None and snapshot["samples"][15]["value"] is None
    assert cli.logit_snapshot(values, 33)["selected_logit"] is None
    small = cli.logit_snapshot(np.array([1.5], dtype=np.float32), 0)
    assert small["samples"] == [{"token_id": 0, "value": 1.5}] and small["count"] == 1
    json.dumps(snapshot)
