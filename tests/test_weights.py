"""Weights: safetensors I/O, loading by name, the one error that lists everything, random weights."""

import json

import pytest
import torch

from lalamo_b200.config import Lfm2Config
from lalamo_b200.weights import WeightsError, load_weights, open_checkpoint, random_tensors, write_random_model, write_safetensors
from lalamo_b200.weights.safetensors_io import SafetensorsFile, SafetensorsFormatError
from tiny import TINY_A, TINY_B


def test_safetensors_round_trip(tmp_path):
    tensors = {
        "a": torch.randn(3, 5),
        "b": torch.randn(7).to(torch.bfloat16),
        "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
        "empty": torch.zeros(0, 4),
    }
    write_safetensors(tmp_path / "x.safetensors", tensors, metadata={"k": "v"})
    file = SafetensorsFile(tmp_path / "x.safetensors")
    assert sorted(file.names()) == sorted(tensors) and file.metadata == {"k": "v"}
    for name, tensor in tensors.items():
        loaded = file.read(name)
        assert loaded.dtype == tensor.dtype and torch.equal(loaded, tensor)
    # the independent reader of the safetensors package agrees
    from safetensors.torch import load_file

    for name, tensor in load_file(str(tmp_path / "x.safetensors")).items():
        assert torch.equal(tensor, tensors[name])


def test_corrupt_header(tmp_path):
    path = tmp_path / "bad.safetensors"
    path.write_bytes(b"\xff" * 8 + b"{}")
    with pytest.raises(SafetensorsFormatError):
        SafetensorsFile(path)
    path.write_bytes((10).to_bytes(8, "little") + b"not json!!")
    with pytest.raises(SafetensorsFormatError):
        SafetensorsFile(path)


@pytest.mark.parametrize("raw", [TINY_A, TINY_B], ids=["A", "B"])
def test_random_model_loads(tmp_path, raw):
    folder = write_random_model(tmp_path / "m", raw, seed=5)
    assert json.loads((folder / "config.json").read_text()) == raw  # spellings survive
    config = Lfm2Config.from_dict(raw)
    weights = load_weights(folder, config)
    embedding = weights[(("embedding",), "weight")]
    assert embedding.shape == (config.vocab_size, config.hidden_size) and embedding.dtype == torch.bfloat16
    for (path, local), tensor in weights.items():
        if local in ("scale", "conv_weight", "conv_bias", "q_norm", "k_norm"):
            assert tensor.dtype == torch.float32, (path, local)  # stored in 32-bit, stays so
    assert ((("lm_head",), "weight") in weights) == (not config.tie_embedding)
    conv_layer = config.layer_types.index("conv")
    assert weights[(("layers", conv_layer, "mixer"), "conv_weight")].shape == (config.hidden_size, config.conv_kernel_size)
    assert open_checkpoint(folder)[f"model.layers.{conv_layer}.conv.conv.weight"].shape == (config.hidden_size, 1, config.conv_kernel_size)


def test_random_weights_depend_on_seed_and_name_only():
    config = Lfm2Config.from_dict(TINY_A)
    first, again, other = random_tensors(config, 3), random_tensors(config, 3), random_tensors(config, 4)
    assert all(torch.equal(first[name], again[name]) for name in first)
    assert not torch.equal(first["model.embed_tokens.weight"], other["model.embed_tokens.weight"])
    assert not torch.equal(first["model.layers.0.feed_forward.w1.weight"], first["model.layers.0.feed_forward.w3.weight"])
    assert abs(float(first["model.layers.0.operator_norm.weight"].mean()) - 1.0) < 0.05


def test_float32_storage_is_kept(tmp_path):
    folder = write_random_model(tmp_path / "m", TINY_A, seed=1, dtype="float32")
    weights = load_weights(folder, Lfm2Config.from_dict(TINY_A))
    assert all(tensor.dtype == torch.float32 for tensor in weights.values())


def test_one_error_lists_everything(tmp_path):
    config = Lfm2Config.from_dict(TINY_B)
    tensors = random_tensors(config, 0)
    del tensors["model.layers.1.conv.in_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(96)
    tensors["model.layers.2.feed_forward.w2.weight"] = torch.zeros(96, 255)
    tensors["model.embedding_norm.weight"] = torch.zeros(97)
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as info:
        load_weights(tmp_path, config)
    error = info.value
    assert error.missing == ["model.layers.1.conv.in_proj.weight", "lm_head.weight"]
    assert error.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert sorted(name for name, _, _ in error.wrong_shape) == ["model.embedding_norm.weight", "model.layers.2.feed_forward.w2.weight"]
    text = str(error)
    for fragment in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "expected [96, 256], found [96, 255]"):
        assert fragment in text


def test_aliases_and_shards(tmp_path):
    config = Lfm2Config.from_dict(TINY_A)
    tensors = random_tensors(config, 0)
    tensors["model.layers.1.self_attn.o_proj.weight"] = tensors.pop("model.layers.1.self_attn.out_proj.weight")
    tensors["model.layers.1.self_attn.q_norm.weight"] = tensors.pop("model.layers.1.self_attn.q_layernorm.weight")
    taps = tensors.pop("model.layers.0.conv.conv.weight")
    tensors["model.layers.0.conv.conv1d.weight"] = taps.reshape(64, 3, 1)  # the other depthwise layout
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    names = sorted(tensors)
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {name: tensors[name] for name in names[:20]})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {name: tensors[name] for name in names[20:]})
    weights = load_weights(tmp_path, config)
    assert torch.equal(weights[(("layers", 0, "mixer"), "conv_weight")], taps.reshape(64, 3))
    assert (("layers", 1, "mixer"), "out_proj") in weights


def test_integer_storage_for_a_matrix_is_refused(tmp_path):
    config = Lfm2Config.from_dict(TINY_A)
    tensors = random_tensors(config, 0)
    tensors["model.embed_tokens.weight"] = torch.zeros(512, 64, dtype=torch.int32)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as info:
        load_weights(tmp_path, config)
    assert info.value.wrong_dtype == [("model.embed_tokens.weight", "I32")]
