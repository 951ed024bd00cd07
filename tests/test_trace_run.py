"""`bin/trace_run` as a user runs it: a subprocess, JSON lines in, logits files out."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

import tiny_configs
from helpers import plain_logits, random_prompts

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOLERANCE = {"float32": 1e-4, "bfloat16": 2e-2}


def replay(folder, dtype, steps, out, max_tokens):
    lines = "".join(json.dumps(step) + "\n" for step in steps)
    done = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
                           "--max-tokens", str(max_tokens)], input=lines, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert done.stdout.split() == [word for step in steps for word in ("done", str(step["step"]))]

    def logits(step, vocab):
        return torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, vocab).copy())

    return logits


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16")])
def test_replay_in_three_cuttings(tmp_path, which, dtype):
    vocab = tiny_configs.CONFIGS[which]["vocab_size"]
    # bfloat16 runs on a folder stored in 32-bit too: replay does not ask what the folder declares.
    folder = tiny_configs.write_tiny(str(tmp_path), which)
    requests = dict(zip("abc", random_prompts(vocab, [70, 41, 100], seed=3)))
    steps, number = [], 0
    expect = []     # (step, rows of (request, position))
    # 1. each request alone and whole
    for name, tokens in requests.items():
        steps.append({"step": number, "entries": [{"id": name + "1", "tokens": tokens, "want": list(range(len(tokens)))}], "end": [name + "1"]})
        expect.append((number, [(name, position) for position in range(len(tokens))]))
        number += 1
    # 2. the last 32 tokens one by one
    tokens = requests["c"]
    steps.append({"step": number, "entries": [{"id": "c2", "tokens": tokens[:-32], "want": []}], "end": []})
    number += 1
    for position in range(len(tokens) - 32, len(tokens)):
        steps.append({"step": number, "entries": [{"id": "c2", "tokens": [tokens[position]], "want": [0]}],
                      "end": ["c2"] if position == len(tokens) - 1 else []})
        expect.append((number, [("c", position)]))
        number += 1
    # 3. a batch of unequal lengths; shorter requests end earlier; then a second batch on the slots given back
    for wave in range(2):
        cut = {"a": 60, "b": 36, "c": 90} if wave == 0 else {"a": 1, "b": 40, "c": 64}
        live = ["a", "b", "c"]
        tag = str(3 + wave)
        steps.append({"step": number, "entries": [{"id": n + tag, "tokens": requests[n][: cut[n]], "want": [cut[n] - 1]} for n in live], "end": []})
        expect.append((number, [(n, cut[n] - 1) for n in live]))
        number += 1
        offset = 0
        while live:
            going = [n for n in live if cut[n] + offset < len(requests[n])]
            ended = [n + tag for n in live if cut[n] + offset + 1 >= len(requests[n])]
            if going:
                steps.append({"step": number, "entries": [{"id": n + tag, "tokens": [requests[n][cut[n] + offset]], "want": [0]} for n in going],
                              "end": ended})
                expect.append((number, [(n, cut[n] + offset) for n in going]))
            else:
                steps.append({"step": number, "entries": [], "end": ended})
            number += 1
            live = [n for n in going if n + tag not in ended]
            offset += 1
    out = str(tmp_path / "out")
    logits = replay(folder, dtype, steps, out, max_tokens=64 * 5)
    plain = {name: plain_logits(folder, tokens, bf16=dtype == "bfloat16") for name, tokens in requests.items()}
    for step, rows in expect:
        found = logits(step, vocab)
        assert found.shape[0] == len(rows)
        wanted = torch.stack([plain[name][position] for name, position in rows])
        assert float((found.double() - wanted.double()).abs().max() / wanted.abs().max()) < TOLERANCE[dtype], (step, rows[:2])
    assert not os.path.exists(os.path.join(out, f"{len(requests)}.f32"))    # a step that wants nothing writes nothing
