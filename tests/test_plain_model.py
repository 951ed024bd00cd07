"""The plain implementation against itself and against committed values (no GPU)."""
import json
import os

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "plain_tiny.json")


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {which: tiny_configs.write_tiny(str(root), which) for which in ("A", "B")}


def test_causality_and_prefix_consistency(folders):
    for which in ("A", "B"):
        config = plain_model.read_plain_config(folders[which])
        weights = plain_model.read_plain_weights(folders[which])
        tokens = np.random.default_rng(1).integers(0, config.vocab_size, size=40).tolist()
        whole = plain_model.forward_logits(config, weights, tokens)
        prefix = plain_model.forward_logits(config, weights, tokens[:23])
        assert torch.allclose(whole[:23], prefix, atol=1e-5, rtol=1e-5)
        changed = list(tokens)
        changed[30] = (changed[30] + 1) % config.vocab_size
        assert torch.allclose(plain_model.forward_logits(config, weights, changed)[:30], whole[:30], atol=1e-6)


def test_double_precision_agrees(folders):
    config = plain_model.read_plain_config(folders["B"])
    weights = plain_model.read_plain_weights(folders["B"])
    tokens = list(range(3, 60))
    single = plain_model.forward_logits(config, weights, tokens)
    double = plain_model.forward_logits(config, {k: v.double() for k, v in weights.items()}, tokens)
    assert float((single.double() - double).abs().max() / double.abs().max()) < 1e-5


def test_rope_is_a_rotation_and_relative():
    cos, sin = plain_model.rope_tables(32, 1e6, 64)
    x = torch.randn(64, 3, 32)
    y = plain_model.apply_rope(x, cos, sin, plain_model.no_rounding)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)
    assert torch.equal(y[0], x[0])
    q = plain_model.apply_rope(x[:1].expand(64, 3, 32).contiguous(), cos, sin, plain_model.no_rounding)
    assert torch.allclose((q[5] * q[9]).sum(-1), (q[25] * q[29]).sum(-1), atol=1e-3)


def test_greedy_rule():
    nan = float("nan")
    assert plain_model.greedy_token([1.0, 3.0, 3.0, 2.0]) == 2
    assert plain_model.greedy_token([nan, -float("inf"), nan]) == 1
    assert plain_model.greedy_token([-0.0, 0.0, -0.0]) == 1
    with pytest.raises(ValueError):
        plain_model.greedy_token([nan, nan])


def test_committed_values(folders):
    with open(GOLDEN) as handle:
        golden = json.load(handle)
    for which in ("A", "B"):
        config = plain_model.read_plain_config(folders[which])
        weights = plain_model.read_plain_weights(folders[which])
        entry = golden[which]
        logits = plain_model.forward_logits(config, weights, entry["tokens"])
        assert np.allclose(logits[-1, :16].numpy(), entry["last_logits_first_16"], atol=2e-5, rtol=0)
        assert int(logits[-1].argmax()) == entry["last_argmax"]
        assert plain_model.greedy_generate(config, weights, entry["tokens"], 6) == entry["greedy_6"]
