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


def rewrite(folder, change):
    tensors = {name: load_tensor(entry) for name, entry in read_catalog(folder).items()}
    change(tensors)
    write_file(folder / "model.safetensors", tensors)
    return tensors


def test_extra_tensors_are_auxiliary_unless_strict(tmp_path):
    """libmir classes a stored tensor that no role asks for as auxiliary; older Llama folders carry
    rotary_emb.inv_freq buffers.  They are ignored (and remembered); with strict=True they are the error."""
    folder = write_model_folder(tmp_path, TINY_A, seed=0, dtype="float32")
    rewrite(folder, lambda t: t.update({"model.layers.0.self_attn.rotary_emb.inv_freq": torch.zeros(8)}))
    model = cpu_model(TINY_A, folder)
    load_into(model, folder)
    assert model.ignored_tensors == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    with pytest.raises(WeightsError) as info:
        load_into(cpu_model(TINY_A, folder), folder, strict=True)
    assert info.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"] and not info.value.missing


@pytest.mark.parametrize("fused_name", ["qkv_proj", "query_key_value"])
def test_fused_qkv_is_split_by_rows(tmp_path, fused_name):
    """A checkpoint that stores [Wq; Wk; Wv] (and the biases) as one tensor binds to the same weights as the
    folder with separate tensors."""
    folder = write_model_folder(tmp_path / "split", TINY_C, seed=0, dtype="float32")
    split = cpu_model(TINY_C, folder)
    load_into(split, folder)
    fused_folder = write_model_folder(tmp_path / "fused", TINY_C, seed=0, dtype="float32")

    def fuse(tensors):
        for layer in range(TINY_C["num_hidden_layers"]):
            stem = f"model.layers.{layer}.self_attn."
            for kind in ("weight", "bias"):
                parts = [tensors.pop(f"{stem}{p}_proj.{kind}") for p in "qkv"]
                tensors[f"{stem}{fused_name}.{kind}"] = torch.cat(parts, dim=0)
    rewrite(fused_folder, fuse)
    fused = cpu_model(TINY_C, fused_folder)
    assert fused.spec == split.spec                       # the bias was discovered from the fused tensor
    load_into(fused, fused_folder)
    for a, b in zip(split.blocks, fused.blocks):
        assert torch.equal(a.mixer.w_qkv, b.mixer.w_qkv) and torch.equal(a.mixer.b_qkv, b.mixer.b_qkv)
        assert torch.equal(a.mixer.w_o, b.mixer.w_o)


def test_fused_and_separate_together_and_a_wrong_fused_shape_are_errors(tmp_path):
    folder = write_model_folder(tmp_path, TINY_A, seed=0, dtype="float32")

    def add_fused(tensors):
        stem = "model.layers.1.self_attn."
        tensors[stem + "qkv_proj.weight"] = torch.cat([tensors[stem + f"{p}_proj.weight"] for p in "qkv"], dim=0)
    rewrite(folder, add_fused)
    with pytest.raises(WeightsError, match="fused and separate") as info:
        load_into(cpu_model(TINY_A, folder), folder)
    assert "model.layers.1.self_attn.k_proj.weight" in str(info.value)

    def only_fused_but_short(tensors):
        stem = "model.layers.1.self_attn."
        for p in "qkv":
            del tensors[stem + f"{p}_proj.weight"]
        tensors[stem + "qkv_proj.weight"] = tensors[stem + "qkv_proj.weight"][:-1]
    rewrite(folder, only_fused_but_short)
    with pytest.raises(WeightsError, match=r"qkv_proj.weight: expected \[128, 64\]") as info:
        load_into(cpu_model(TINY_A, folder), folder)
    assert len(info.value.wrong_shape) == 3 and not info.value.missing


def test_tensors_stored_in_out_are_transposed(tmp_path):
    """[in, out] tensors are recognised by their shape (libmir: transposes_last_two); a square tensor is taken as
    stored."""
    folder = write_model_folder(tmp_path / "plain", TINY_A, seed=0, dtype="float32")
    plain = cpu_model(TINY_A, folder)
    load_into(plain, folder)
    other = write_model_folder(tmp_path / "swapped", TINY_A, seed=0, dtype="float32")

    def swap(tensors):
        for name in list(tensors):
            if name.endswith(("mlp.down_proj.weight", "mlp.gate_proj.weight", "self_attn.k_proj.weight", "lm_head.weight")):
                tensors[name] = tensors[name].t().contiguous()
    rewrite(other, swap)
    swapped = cpu_model(TINY_A, other)
    load_into(swapped, other)
    for a, b in zip(plain.blocks, swapped.blocks):
        assert torch.equal(a.feed_forward.w_gate_up, b.feed_forward.w_gate_up)
        assert torch.equal(a.feed_forward.w_down, b.feed_forward.w_down) and torch.equal(a.mixer.w_qkv, b.mixer.w_qkv)
    assert torch.equal(plain.head, swapped.head)
