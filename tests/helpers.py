"""Shared by the tests: building engines on tiny folders, replaying requests in several cuttings."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

import plain_model
from tau_rs_b200 import Engine, StepEntry, load_model


def random_prompts(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=length).tolist() for length in lengths]


def plain_logits(folder: str, tokens: Sequence[int], bf16: bool = False) -> torch.Tensor:
    config = plain_model.read_plain_config(folder)
    weights = plain_model.read_plain_weights(folder)
    if bf16:
        weights = {name: plain_model.bfloat16_rounding(value) if value.dim() > 1 else value for name, value in weights.items()}
    rounding = plain_model.bfloat16_rounding if bf16 else plain_model.no_rounding
    return plain_model.forward_logits(config, weights, tokens, rounding)


def engine_for(folder: str, dtype: str, device, max_tokens: int = 4096) -> Engine:
    device = torch.device(device) if isinstance(device, str) and device != "gpu" else device
    return Engine(load_model(folder, dtype, device), max_tokens)


def run_whole(engine: Engine, tokens: Sequence[int]) -> torch.Tensor:
    """One request alone, all tokens in one step, logits everywhere."""
    slot = engine.open_sequence()
    try:
        logits = engine.step([StepEntry(slot, list(tokens), list(range(len(tokens))))])
        return logits.float().cpu().clone()
    finally:
        engine.close_sequence(slot)


def run_tail_stepwise(engine: Engine, tokens: Sequence[int], tail: int) -> torch.Tensor:
    """The prefix in one step, the last `tail` tokens one by one; logits of the tail."""
    tail = min(tail, len(tokens) - 1)
    slot = engine.open_sequence()
    rows = []
    try:
        prefix = list(tokens[: len(tokens) - tail])
        engine.step([StepEntry(slot, prefix, [])])
        for token in tokens[len(tokens) - tail :]:
            rows.append(engine.step([StepEntry(slot, [token], [0])]).float().cpu().clone())
        return torch.cat(rows, dim=0)
    finally:
        engine.close_sequence(slot)


def run_batched(engine: Engine, requests: Sequence[Sequence[int]], prompt_lengths: Sequence[int]) -> List[torch.Tensor]:
    """Requests start together: prompts of the given lengths in one step, then one token each until each
    request's tokens run out; a request that ends gives its slot back at once.  Returns for each request
    the logits at its last prompt token and at every later token."""
    slots = [engine.open_sequence() for _ in requests]
    live = list(range(len(requests)))
    out: List[List[torch.Tensor]] = [[] for _ in requests]
    try:
        entries = [StepEntry(slots[i], list(requests[i][: prompt_lengths[i]]), [prompt_lengths[i] - 1]) for i in live]
        logits = engine.step(entries).float().cpu()
        for row, i in enumerate(live):
            out[i].append(logits[row].clone())
        cursor = {i: prompt_lengths[i] for i in live}
        while True:
            for i in list(live):
                if cursor[i] >= len(requests[i]):
                    engine.close_sequence(slots[i])
                    live.remove(i)
            if not live:
                break
            entries = [StepEntry(slots[i], [requests[i][cursor[i]]], [0]) for i in live]
            logits = engine.step(entries).float().cpu()
            for row, i in enumerate(live):
                out[i].append(logits[row].clone())
                cursor[i] += 1
        return [torch.stack(rows) for rows in out]
    finally:
        for i in live:
            engine.close_sequence(slots[i])


def relative_error(found: torch.Tensor, wanted: torch.Tensor) -> float:
    """Largest absolute difference over the largest absolute wanted value."""
    return float((found.double() - wanted.double()).abs().max() / wanted.double().abs().max())


# ---- a toy architecture whose attention layers all have a window (so that their cache gives old pages back) ----------
def window_spec(config):
    from tau_rs_b200.config import AttentionSpec, BlockSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry, SwiGLUSpec

    hidden = config["hidden_size"]
    norm = NormSpec(width=hidden, eps=config["eps"])
    position = PositionSpec(rotary_dim=16, theta=1000.0, max_positions=config["max_positions"])
    first = AttentionSpec(hidden=hidden, n_heads=4, n_kv_heads=2, head_dim=16, bias=False, softmax_scale=0.25,
                          qk_norm=NormSpec(width=16, eps=config["eps"]), position=position, window=config["window"])
    second = AttentionSpec(hidden=hidden, n_heads=2, n_kv_heads=1, head_dim=32, bias=True, softmax_scale=32 ** -0.5, qk_norm=None,
                           position=position, window=config["window"] // 2)
    feed = SwiGLUSpec(hidden=hidden, intermediate=config["intermediate_size"])
    blocks = (BlockSpec("toy.layers.0", first, feed, norm, norm), BlockSpec("toy.layers.1", second, feed, norm, norm))
    schedule = (ScheduleEntry(layer=0, cache_group="wide", cache_layer=0), ScheduleEntry(layer=1, cache_group="narrow", cache_layer=0))
    return ModelSpec(architecture="ToyWindowForCausalLM", vocab_size=config["vocab_size"], hidden=hidden, max_positions=config["max_positions"],
                     embedding_name="toy.embed.weight", blocks=blocks, schedule=schedule, final_norm=norm,
                     final_norm_name="toy.norm.weight", head_name="toy.head.weight", tie_head=True)


WINDOW_CONFIG = {"architectures": ["ToyWindowForCausalLM"], "model_type": "toy_window", "hidden_size": 32, "intermediate_size": 48,
                 "vocab_size": 53, "max_positions": 1024, "eps": 1e-5, "window": 70}


def windowed_cache_matches_whole_prompt(folder, dtype, device, tolerance):
    """A sequence of 600 tokens through an engine whose cache holds 4 pages (256 positions), in chunks and single tokens, against
    the same tokens in one step through an engine with room for all of them: the pages that fell out of the windows were given
    back and taken again, and nothing that a query may see was lost."""
    import numpy as np

    from tau_rs_b200 import Engine, StepEntry, load_model

    model = load_model(folder, dtype, device)
    tokens = np.random.default_rng(3).integers(0, WINDOW_CONFIG["vocab_size"], size=600).tolist()
    roomy = Engine(model, 64 * 10)
    slot = roomy.open_sequence()
    wanted = roomy.step([StepEntry(slot, tokens, list(range(len(tokens))))]).cpu().clone()
    roomy.close_sequence(slot)
    tight = Engine(model, 64 * 4)
    assert tight.max_sequence_tokens == WINDOW_CONFIG["max_positions"]
    slot = tight.open_sequence()
    found, position = [], 0
    for count in [50, 1, 1, 64, 30, 1, 1, 1, 50, 50, 50, 64, 1, 50, 50, 50, 36] + [1] * 50:
        piece = tokens[position : position + count]
        found.append(tight.step([StepEntry(slot, piece, list(range(len(piece))))]).cpu().clone())
        position += len(piece)
        tight.cache.check()
        assert len(tight.cache.kv["wide"].held[slot]) <= 3 and len(tight.cache.kv["narrow"].held[slot]) <= 3
    assert position == 600
    tight.close_sequence(slot)
    tight.cache.check()
    import torch

    found = torch.cat(found)
    assert relative_error(found, wanted) < tolerance


# ---- models of real widths, drawn on the device ----------------------------------------------------------------------
def drawn_models(config_json: dict, seed: int, norm_jitter: float, dtypes: Sequence[str]):
    """Draws the weights of `config_json` once on the GPU (every value one that bfloat16 holds), builds one model per
    dtype of `dtypes` from the same values (a float32 model holds the bfloat16 values widened), and returns
    `(plain config, plain weights on the CPU in float32, {dtype: model})`.  Nothing touches a disk."""
    from tau_rs_b200.config.registry import architecture_for
    from tau_rs_b200.parts import DecoderModel
    from tau_rs_b200.weights import device_dtype, random_tensors

    entry = architecture_for(config_json)
    spec = entry.build_spec(entry.parse_config(config_json))
    device = torch.device("cuda:0")
    models = {dtype: DecoderModel(spec, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], device) for dtype in dtypes}
    plain_weights = {}
    specs = next(iter(models.values())).tensor_specs()
    for name, tensor, tensor_spec in random_tensors(specs, seed, norm_jitter, device=device, dtype_of=lambda _: torch.bfloat16):
        plain_weights[name] = tensor.float().cpu()
        for dtype, model in models.items():
            model.assign(name, tensor.to(device_dtype(tensor_spec, model.dtype)))
    for model in models.values():
        model.finalize_weights()
    heads = config_json["num_attention_heads"]
    plain_config = plain_model.PlainConfig(
        vocab_size=config_json["vocab_size"], hidden_size=config_json["hidden_size"], intermediate_size=config_json["intermediate_size"],
        num_hidden_layers=config_json["num_hidden_layers"], num_attention_heads=heads,
        num_key_value_heads=config_json.get("num_key_value_heads", heads), head_dim=config_json.get("head_dim", config_json["hidden_size"] // heads),
        attention_bias=config_json.get("attention_bias", False), rms_norm_eps=config_json["rms_norm_eps"], rope_theta=config_json["rope_theta"],
        max_position_embeddings=config_json["max_position_embeddings"], tie_word_embeddings=config_json.get("tie_word_embeddings", False))
    return plain_config, plain_weights, models


def plain_rows(plain_config, plain_weights, tokens: Sequence[int], rows: Sequence[int], bf16: bool) -> torch.Tensor:
    """The plain implementation's logits of `tokens` at the positions `rows`."""
    rounding = plain_model.bfloat16_rounding if bf16 else plain_model.no_rounding
    return plain_model.forward_logits(plain_config, plain_weights, tokens, rounding, rows=rows)
