"""Safetensors reading, the weight contract and the random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

import plain_model
import tiny_configs
from tau_rs_b200.config import WeightError, spec_from_config_json
from tau_rs_b200.config.errors import MissingFile, ModelLoadError
from tau_rs_b200.parts import DecoderModel
from tau_rs_b200.weights import SafetensorsFolder, load_weights, write_random_model, write_safetensors


def model_for(which, dtype=torch.float32):
    return DecoderModel(spec_from_config_json(tiny_configs.CONFIGS[which]), dtype, torch.device("cpu"))


def rewrite(folder, change):
    """Reads every tensor of a folder, lets `change` edit the dict, writes it back."""
    found = SafetensorsFolder(folder)
    tensors = {name: found.read(name).clone() for name in found.tensors}
    found.close()
    change(tensors)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())


def test_random_folder_reads_back(tmp_path):
    path = tiny_configs.write_tiny(str(tmp_path), "B")
    model = model_for("B")
    load_weights(model, path, torch.float32, torch.device("cpu"))
    assert model.embedding.shape == (500, 96) and model.head.shape == (500, 96) and model.head is not model.embedding
    attention = model.blocks[1].mixer
    assert attention.qkv.weight.shape == ((8 + 2) * 32, 96) and attention.qkv.bias.shape == (320,)
    assert attention.q_norm.weight.dtype == torch.float32 and model.blocks[0].feed_forward.gate_up.weight.shape == (448, 96)
    plain = plain_model.read_plain_weights(path)
    assert torch.equal(attention.qkv.weight[256:288], plain["model.layers.1.self_attn.k_proj.weight"])
    assert torch.equal(model.blocks[2].feed_forward.gate_up.weight[224:], plain["model.layers.2.mlp.up_proj.weight"])
    with open(os.path.join(path, "config.json")) as handle:
        assert json.load(handle)["torch_dtype"] == "float32"


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    first = tiny_configs.write_tiny(str(tmp_path / "one"), "A")
    second = tiny_configs.write_tiny(str(tmp_path / "two"), "A")
    a, b = plain_model.read_plain_weights(first), plain_model.read_plain_weights(second)
    assert all(torch.equal(a[name], b[name]) for name in a)
    write_random_model(str(tmp_path / "other"), tiny_configs.TINY_A, seed=5, norm_jitter=0.1)
    c = plain_model.read_plain_weights(str(tmp_path / "other"))
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert abs(float(a["model.embed_tokens.weight"].std()) - 0.02) < 0.002
    assert abs(float(a["model.norm.weight"].mean()) - 1.0) < 0.1 and float(a["model.norm.weight"].std()) > 0.03
    assert "lm_head.weight" not in a     # tied


def test_bfloat16_storage_and_dtype_rules(tmp_path):
    path = tiny_configs.write_tiny(str(tmp_path), "A", "bfloat16")
    found = SafetensorsFolder(path)
    assert {info.dtype for info in found.tensors.values()} == {"BF16"}
    model = model_for("A", torch.bfloat16)
    load_weights(model, path, torch.bfloat16, torch.device("cpu"))
    assert model.embedding.dtype == torch.bfloat16 and model.head is model.embedding
    assert model.final_norm.weight.dtype == torch.float32           # vectors are kept in 32-bit
    assert model.blocks[0].mixer.position.cos.dtype == torch.float32


def test_one_error_lists_everything_wrong(tmp_path):
    path = tiny_configs.write_tiny(str(tmp_path), "B")

    def damage(tensors):
        del tensors["model.layers.0.self_attn.q_norm.weight"]
        del tensors["model.layers.2.mlp.down_proj.weight"]
        tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(32, 95)
        tensors["model.layers.7.extra.weight"] = torch.zeros(3)
        tensors["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)

    rewrite(path, damage)
    with pytest.raises(WeightError) as error:
        load_weights(model_for("B"), path, torch.float32, torch.device("cpu"))
    assert error.value.missing == ["model.layers.0.self_attn.q_norm.weight", "model.layers.2.mlp.down_proj.weight"]
    assert error.value.unexpected == ["model.layers.7.extra.weight"]
    assert error.value.wrong_shape == [("model.layers.1.self_attn.k_proj.weight", (32, 95), (32, 96))]
    assert error.value.wrong_dtype == [("model.norm.weight", "I32")]
    text = str(error.value)
    for fragment in ("missing tensors (2)", "unexpected tensors (1)", "is [32, 95], expected [32, 96]", "model.norm.weight is I32"):
        assert fragment in text


def test_head_falls_back_to_the_embedding_and_tied_models_ignore_a_head(tmp_path):
    untied = tiny_configs.write_tiny(str(tmp_path / "u"), "B")
    rewrite(untied, lambda tensors: tensors.pop("lm_head.weight"))
    model = model_for("B")
    load_weights(model, untied, torch.float32, torch.device("cpu"))
    assert torch.equal(model.head, model.embedding)
    tied = tiny_configs.write_tiny(str(tmp_path / "t"), "A")
    rewrite(tied, lambda tensors: tensors.update({"lm_head.weight": torch.zeros(256, 64)}))
    model = model_for("A")
    load_weights(model, tied, torch.float32, torch.device("cpu"))
    assert model.head is model.embedding


def test_sharded_folders_and_broken_files(tmp_path):
    path = tiny_configs.write_tiny(str(tmp_path), "A")
    found = SafetensorsFolder(path)
    tensors = {name: found.read(name).clone() for name in found.tensors}
    found.close()
    os.remove(os.path.join(path, "model.safetensors"))
    names = sorted(tensors)
    write_safetensors(os.path.join(path, "model-00001-of-00002.safetensors"), [(n, tensors[n]) for n in names[:5]])
    write_safetensors(os.path.join(path, "model-00002-of-00002.safetensors"), [(n, tensors[n]) for n in names[5:]])
    load_weights(model_for("A"), path, torch.float32, torch.device("cpu"))
    write_safetensors(os.path.join(path, "model-00003.safetensors"), [(names[0], tensors[names[0]])])
    with pytest.raises(ModelLoadError) as error:
        SafetensorsFolder(path)
    assert "appears in" in str(error.value)
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(MissingFile):
        SafetensorsFolder(str(empty))
    (empty / "model.safetensors").write_bytes(b"\xff" * 12)
    with pytest.raises(ModelLoadError):
        SafetensorsFolder(str(empty))


def test_the_counter_based_stream():
    """Philox4x32-10 against its published known answer for a counter and key of zero, and
    the normal values against a double-precision Box-Muller of the same words; a tensor's values depend on the seed and
    its name only, and a tensor drawn in pieces equals the tensor drawn whole."""
    import numpy as np

    from tau_rs_b200.weights.random_init import _draw_on_host, philox4x32, standard_normals, stream_key

    def words(counter0, key0, key1):
        return [int(word[0]) for word in philox4x32(np.array([counter0], dtype=np.uint64), key0, key1)]

    assert words(0, 0, 0) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    key = stream_key(0, "model.norm.weight")
    assert key != stream_key(1, "model.norm.weight") and key != stream_key(0, "model.norm.weigh")
    values = standard_normals(400_003, *key)
    assert values.dtype == np.float32 and np.isfinite(values).all()
    assert abs(float(values.mean())) < 0.01 and abs(float(values.std()) - 1.0) < 0.01
    assert abs(float(((values - values.mean()) ** 4).mean() / values.var() ** 2) - 3.0) < 0.05
    w0, w1, w2, w3 = philox4x32(np.arange(2000, dtype=np.uint64), *key)
    for first, (radius_word, angle_word) in ((0, (w0, w1)), (2, (w2, w3))):
        u = ((radius_word >> np.uint64(9)).astype(np.float64) + 0.5) * 2.0 ** -23
        angle = ((angle_word >> np.uint64(9)).astype(np.float64) + 0.5) * 2.0 ** -23 * 2 * np.pi
        radius = np.sqrt(-2 * np.log(u))
        assert np.abs(values[first:8000:4] - radius * np.cos(angle)).max() < 2e-6
        assert np.abs(values[first + 1:8000:4] - radius * np.sin(angle)).max() < 2e-6
    assert np.array_equal(standard_normals(1000, *key, first_block=25), values[100:1100])
    import tau_rs_b200.weights.random_init as random_init

    whole = _draw_on_host(10_001, *key, 0.02, 0.0)
    old = random_init._HOST_CHUNK
    try:
        random_init._HOST_CHUNK = 4096
        assert np.array_equal(_draw_on_host(10_001, *key, 0.02, 0.0), whole)
    finally:
        random_init._HOST_CHUNK = old
