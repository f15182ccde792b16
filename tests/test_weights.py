"""Safetensors reading/writing, binding by name, the one error that lists everything, random weights (no GPU)."""

import json

import pytest
import torch

from libmir_b200 import WeightsError, build_spec
from libmir_b200.models.decoder import DecoderModel
from libmir_b200.parts.base import BuildEnv
from libmir_b200.weights import (load_into, load_tensor, match, read_catalog, write_file, write_model_folder)
from tiny_configs import TINY_A, TINY_B, TINY_C


def cpu_model(config, folder=None, dtype=torch.float32):
    catalog = None if folder is None else {n: e.shape for n, e in read_catalog(folder).items()}
    return DecoderModel(build_spec(config, catalog), BuildEnv(dtype, torch.device("cpu")))


def test_file_round_trip_all_dtypes(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32),
               "d": torch.randn(2, 2).to(torch.float16), "empty": torch.zeros(0, 4)}
    write_file(tmp_path / "x.safetensors", tensors, {"note": "test"})
    catalog = read_catalog(tmp_path)
    assert set(catalog) == set(tensors)
    for name, tensor in tensors.items():
        loaded = load_tensor(catalog[name])
        assert loaded.dtype == tensor.dtype and loaded.shape == tensor.shape and torch.equal(loaded, tensor)


def test_random_folder_is_seeded_and_complete(tmp_path):
    first = write_model_folder(tmp_path / "a", TINY_B, seed=3, dtype="bfloat16")
    again = write_model_folder(tmp_path / "b", TINY_B, seed=3, dtype="bfloat16")
    other = write_model_folder(tmp_path / "c", TINY_B, seed=4, dtype="bfloat16")
    a, b, c = (read_catalog(f) for f in (first, again, other))
    assert json.loads((first / "config.json").read_text()) == TINY_B
    assert "lm_head.weight" not in a                      # tied head shares the embedding
    assert "model.layers.2.self_attn.q_norm.weight" in a
    for name in a:
        assert torch.equal(load_tensor(a[name]), load_tensor(b[name]))
    weight = "model.layers.0.mlp.down_proj.weight"
    assert not torch.equal(load_tensor(a[weight]), load_tensor(c[weight]))
    values = load_tensor(a[weight]).float()
    assert values.dtype == torch.float32 and abs(values.std().item() - 0.02) < 0.002
    norm = load_tensor(a["model.norm.weight"])
    assert norm.dtype == torch.float32 and torch.all(norm == 1)     # a 32-bit tensor stays 32-bit


def test_load_binds_by_name_and_keeps_dtypes(tmp_path):
    folder = write_model_folder(tmp_path, TINY_C, seed=0, dtype="float32")
    model = cpu_model(TINY_C, folder, torch.bfloat16)
    load_into(model, folder)
    attention = model.blocks[1].mixer
    assert attention.w_qkv.dtype == torch.bfloat16 and attention.w_qkv.shape == ((6 + 2 * 3) * 48, 120)
    assert attention.b_qkv is not None and attention.b_o is not None
    assert model.final_norm.weight.dtype == torch.float32
    assert model.head is not model.embedding and model.head.shape == (515, 120)
    stored = load_tensor(read_catalog(folder)["model.layers.1.self_attn.k_proj.weight"])
    assert torch.equal(attention.w_qkv[6 * 48:9 * 48], stored.to(torch.bfloat16))


def test_wrapping_prefix_is_stripped(tmp_path):
    folder = write_model_folder(tmp_path, TINY_A, seed=0, dtype="float32")
    catalog = read_catalog(folder)
    tensors = {("language_model." + name if name.startswith("model.") else name): load_tensor(entry)
               for name, entry in catalog.items()}
    write_file(folder / "model.safetensors", tensors)
    load_into(cpu_model(TINY_A, folder), folder)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_model_folder(tmp_path, TINY_A, seed=0, dtype="float32")
    tensors = {name: load_tensor(entry) for name, entry in read_catalog(folder).items()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 171)
    tensors["model.norm.weight"] = torch.zeros(65)
    write_file(folder / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as info:
        load_into(cpu_model(TINY_A, folder), folder)
    error = info.value
    assert error.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert error.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(error.wrong_shape) == 2
    text = str(error)
    assert "missing tensors (2)" in text and "unexpected tensors (1)" in text and "wrong shapes (2)" in text
    assert "expected [64, 172], checkpoint has [64, 171]" in text


def test_declared_qk_norm_without_weights_is_an_error(tmp_path):
    folder = write_model_folder(tmp_path, TINY_B, seed=0, dtype="float32")
    tensors = {name: load_tensor(entry) for name, entry in read_catalog(folder).items()
               if "q_norm" not in name and "k_norm" not in name}
    write_file(folder / "model.safetensors", tensors)
    from libmir_b200 import ConfigError
    with pytest.raises(ConfigError, match="no q_norm / k_norm weights"):
        cpu_model(dict(TINY_B, qk_normalization=True), folder)
    # without the declaration the tensors decide: the model is built without q/k-norm
    load_into(cpu_model(TINY_B, folder), folder)


def test_broken_files(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(WeightsError, match="no \\*.safetensors file"):
        read_catalog(tmp_path)
    (tmp_path / "model.safetensors").write_bytes(b"\x10\x00\x00")
    with pytest.raises(WeightsError, match="too short"):
        read_catalog(tmp_path)
    (tmp_path / "model.safetensors").write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightsError, match="exceeds the limit"):
        read_catalog(tmp_path)
