"""Two tiny configurations of dense Qwen3 that differ in every size and option."""
from __future__ import annotations

import os

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "attention_bias": False, "max_position_embeddings": 128, "hidden_act": "silu",
    "sliding_window": None, "use_sliding_window": False, "max_window_layers": 2, "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 8, "num_key_value_heads": 1, "head_dim": 32,
    "intermediate_size": 224, "vocab_size": 500, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "attention_bias": True, "max_position_embeddings": 256, "hidden_act": "silu",
    "eos_token_id": [3, 499], "max_new_tokens": 12,
}
# Wider than a page and longer than a few pages: 5 heads in one group of 5, head_dim 48, odd widths.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48,
    "intermediate_size": 200, "vocab_size": 333, "rope_theta": 50000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "attention_bias": False, "max_position_embeddings": 1024, "hidden_act": "silu",
}
SEEDS = {"A": 0, "B": 1, "C": 2}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
STORAGE = {"A": "bfloat16", "B": "float32", "C": "bfloat16"}


def write_tiny(folder: str, which: str, storage: str = None) -> str:
    from tau_rs_b200.weights import write_random_model

    path = os.path.join(folder, f"tiny_{which}")
    write_random_model(path, CONFIGS[which], seed=SEEDS[which], norm_jitter=0.1, storage=storage or STORAGE[which])
    return path
