"""Configuration, registry and generation settings (no GPU)."""
import json

import pytest

import tiny_configs
from tau_rs_b200.config import (InvalidConfig, Qwen3Config, UnsupportedDType, architecture_for, load_generation_config,
                                metadata_from_json, read_config_json, registered_architectures, spec_from_config_json,
                                validate_run_dtype)
from tau_rs_b200.config.errors import InvalidModelDir, MissingFile

# The fixture of crates/models/src/qwen3.rs:136-156.
REFERENCE_FIXTURE = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 64, "hidden_size": 16,
    "intermediate_size": 32, "num_hidden_layers": 1, "num_attention_heads": 2, "head_dim": 8, "attention_bias": False,
    "num_key_value_heads": 1, "max_position_embeddings": 128, "sliding_window": None, "max_window_layers": 1,
    "tie_word_embeddings": True, "rope_theta": 1000000.0, "rms_norm_eps": 0.000001, "use_sliding_window": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}


def test_reference_fixture_keeps_its_fields():
    config = Qwen3Config.from_json(REFERENCE_FIXTURE)
    assert (config.hidden_size, config.head_dim, config.num_attention_heads, config.num_key_value_heads) == (16, 8, 2, 1)
    assert config.max_position_embeddings == 128 and not config.attention_bias and config.tie_word_embeddings
    assert config.rope_theta == 1e6 and config.rms_norm_eps == 1e-6 and config.declared_dtype == "bfloat16"
    assert Qwen3Config.from_json(config.to_json()) == config


def test_defaults_follow_the_other_keys():
    raw = dict(tiny_configs.TINY_A)
    del raw["head_dim"], raw["num_key_value_heads"], raw["tie_word_embeddings"], raw["attention_bias"]
    config = Qwen3Config.from_json(raw)
    assert config.head_dim == 16 and config.num_key_value_heads == 4
    assert not config.tie_word_embeddings and not config.attention_bias


@pytest.mark.parametrize("change,fragment", [
    ({"hidden_size": None}, "hidden_size"), ({"vocab_size": 0}, "vocab_size"), ({"rms_norm_eps": -1}, "rms_norm_eps"),
    ({"rope_theta": "big"}, "rope_theta"), ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"use_sliding_window": True}, "sliding"), ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"attention_bias": "yes"}, "attention_bias"), ({"num_hidden_layers": 2.5}, "num_hidden_layers"),
])
def test_invalid_values_are_refused(change, fragment):
    raw = dict(tiny_configs.TINY_A)
    for key, value in change.items():
        if value is None:
            raw.pop(key)
        else:
            raw[key] = value
    with pytest.raises(InvalidConfig) as error:
        Qwen3Config.from_json(raw)
    assert fragment in str(error.value)


def test_registry_names_both_keys_for_an_unknown_model():
    assert "Qwen3ForCausalLM" in registered_architectures()
    raw = dict(tiny_configs.TINY_A, architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe")
    with pytest.raises(InvalidConfig) as error:
        architecture_for(raw)
    assert "Qwen3MoeForCausalLM/qwen3_moe" in str(error.value) and "Qwen3ForCausalLM/qwen3" in str(error.value)
    with pytest.raises(InvalidConfig):
        architecture_for(dict(tiny_configs.TINY_A, model_type="qwen2"))
    with pytest.raises(InvalidConfig):
        metadata_from_json({"model_type": "qwen3"})


def test_spec_carries_every_size_to_the_parts():
    spec = spec_from_config_json(tiny_configs.TINY_B)
    assert len(spec.blocks) == 3 and len(spec.schedule) == 3 and spec.vocab_size == 500 and not spec.tie_head
    mixer = spec.blocks[0].mixer
    assert (mixer.n_heads, mixer.n_kv_heads, mixer.head_dim, mixer.bias, mixer.hidden) == (8, 1, 32, True, 96)
    assert mixer.qk_norm.eps == 1e-5 and mixer.qk_norm.width == 32 and mixer.position.theta == 1e6
    assert mixer.position.rotary_dim == 32 and mixer.position.max_positions == 256 and abs(mixer.softmax_scale - 32 ** -0.5) < 1e-12
    assert spec.blocks[2].feed_forward.intermediate == 224 and spec.blocks[2].prefix == "model.layers.2"
    assert [(entry.layer, entry.cache_layer, entry.writes_cache) for entry in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True)]


def test_dtype_gate():
    bf16 = metadata_from_json(dict(tiny_configs.TINY_A, torch_dtype="bfloat16"))
    f32 = metadata_from_json(dict(tiny_configs.TINY_A, dtype="float32"))
    assert validate_run_dtype(bf16, "bf16") == "bfloat16" and validate_run_dtype(bf16, "f32") == "float32"
    assert validate_run_dtype(f32, "float32") == "float32"
    with pytest.raises(UnsupportedDType):
        validate_run_dtype(f32, "bfloat16")
    with pytest.raises(UnsupportedDType):
        validate_run_dtype(bf16, "float16")
    with pytest.raises(InvalidConfig):
        metadata_from_json(dict(tiny_configs.TINY_A, torch_dtype="bfloat16", dtype="float32"))


def test_folder_errors(tmp_path):
    with pytest.raises(InvalidModelDir):
        read_config_json(str(tmp_path / "absent"))
    with pytest.raises(MissingFile):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(InvalidConfig):
        read_config_json(str(tmp_path))


def test_generation_settings(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(tiny_configs.TINY_B))
    settings = load_generation_config(str(tmp_path))
    assert settings.eos_token_ids == (3, 499) and settings.max_new_tokens == 12 and settings.is_eos_token(499)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 5}))
    settings = load_generation_config(str(tmp_path))
    assert settings.eos_token_ids == (5,) and settings.max_new_tokens == 16
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 5, "max_new_tokens": 0}))
    with pytest.raises(InvalidConfig):
        load_generation_config(str(tmp_path))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [-1]}))
    with pytest.raises(InvalidConfig):
        load_generation_config(str(tmp_path))
