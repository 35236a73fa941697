"""Safetensors reading and writing, the loader's one clear error, random weights."""

import json
import struct

import pytest
import torch

import shrike_b200.models  # noqa: F401
from shrike_b200.config import parse_config
from shrike_b200.weights import (
    SafetensorsError, SafetensorsFile, WeightError, expected_tensors, load_weights, random_tensors,
    write_model_folder, write_safetensors,
)
from tests.helpers import make_model_folder, read_weights
from tests.tiny_configs import TINY_A, TINY_B


def test_round_trip_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file

    tensors = {"m": torch.randn(5, 7), "v": torch.randn(9).bfloat16(), "i": torch.arange(6, dtype=torch.int64),
               "h": torch.randn(3, 2).half(), "empty": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "ours.safetensors", tensors, {"note": "x"})
    theirs = load_file(str(tmp_path / "ours.safetensors"))
    save_file(tensors, str(tmp_path / "theirs.safetensors"))
    ours = SafetensorsFile(tmp_path / "theirs.safetensors")
    for name, tensor in tensors.items():
        assert torch.equal(theirs[name], tensor)
        assert torch.equal(ours.tensor(name), tensor)
        assert ours.shape(name) == tuple(tensor.shape) and ours.dtype(name) == tensor.dtype


def test_broken_files_are_refused(tmp_path):
    path = tmp_path / "bad.safetensors"
    path.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="shorter"):
        SafetensorsFile(path)
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(path)
    header = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="bad offsets"):
        SafetensorsFile(path)
    header = json.dumps({"t": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="dtype"):
        SafetensorsFile(path)


def test_expected_names_are_the_reference_state_dict_keys():
    names = set(expected_tensors(parse_config(TINY_A)))
    assert "model.embed_tokens.weight" in names and "model.norm.weight" in names and "lm_head.weight" in names
    for stem in ("self_attn.q_proj.weight", "self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.weight",
                 "self_attn.o_proj.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight",
                 "input_layernorm.weight", "post_attention_layernorm.weight"):
        assert f"model.layers.1.{stem}" in names
    assert "model.layers.0.self_attn.o_proj.bias" not in names
    assert len(names) == 3 + 2 * 12


def test_loader_lists_missing_unexpected_and_wrong_shapes_at_once(tmp_path):
    folder = make_model_folder(tmp_path, "B")
    weights = read_weights(folder)
    del weights["model.layers.1.mlp.up_proj.weight"]
    del weights["model.norm.weight"]
    weights["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    weights["model.layers.2.self_attn.k_proj.bias"] = torch.zeros(97)
    write_safetensors(folder / "model.safetensors", weights)
    with pytest.raises(WeightError) as info:
        load_weights(folder, parse_config(TINY_B), torch.float32, "cpu")
    error = info.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert error.wrong_shape == [("model.layers.2.self_attn.k_proj.bias", (96,), (97,))]
    text = str(error)
    assert "missing (2)" in text and "unexpected (1)" in text and "expected [96] got [97]" in text


def test_untied_model_needs_its_head_and_tied_model_aliases(tmp_path):
    folder = make_model_folder(tmp_path, "B")
    weights = read_weights(folder)
    del weights["lm_head.weight"]
    write_safetensors(folder / "model.safetensors", weights)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(folder, parse_config(TINY_B), torch.float32, "cpu")
    tied = make_model_folder(tmp_path, "A")
    loaded = load_weights(tied, parse_config(TINY_A), torch.float32, "cpu")
    assert loaded["lm_head.weight"].data_ptr() == loaded["model.embed_tokens.weight"].data_ptr()


def test_duplicate_names_across_files_and_missing_files(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    weights = read_weights(folder)
    write_safetensors(folder / "extra.safetensors", {"model.norm.weight": weights["model.norm.weight"]})
    with pytest.raises(WeightError, match="more than one file"):
        load_weights(folder, parse_config(TINY_A), torch.float32, "cpu")
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_weights(empty, parse_config(TINY_A), torch.float32, "cpu")


def test_kept_precision(tmp_path):
    config = parse_config(TINY_A)
    stored32 = make_model_folder(tmp_path, "A", "float32")
    as_bf16 = load_weights(stored32, config, torch.bfloat16, "cpu")
    assert as_bf16["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16   # matrices feed the tensor cores
    assert as_bf16["model.norm.weight"].dtype == torch.float32                        # stored in 32-bit: stays
    assert as_bf16["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32
    stored16 = make_model_folder(tmp_path, "A", "bfloat16")
    kept = load_weights(stored16, config, torch.bfloat16, "cpu")
    assert all(t.dtype == torch.bfloat16 for t in kept.values())
    widened = load_weights(stored16, config, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in widened.values())


def test_integer_tensors_become_int32():
    from shrike_b200.weights.loader import kept_dtype

    assert kept_dtype(torch.int64, 1, torch.bfloat16) == torch.int32
    assert kept_dtype(torch.uint8, 2, torch.float32) == torch.int32


def test_random_weights_are_reproducible_and_distributed_as_said(tmp_path):
    config = parse_config(TINY_B)
    one, two, other = random_tensors(config, 1), random_tensors(config, 1), random_tensors(config, 2)
    assert all(torch.equal(one[k], two[k]) for k in one)
    assert not torch.equal(one["model.norm.weight"], other["model.norm.weight"])
    matrix = one["model.embed_tokens.weight"]
    assert abs(float(matrix.std()) - 0.02) < 1e-3 and abs(float(matrix.mean())) < 1e-3
    norm = torch.cat([v for k, v in one.items() if k.endswith("norm.weight")])
    assert abs(float(norm.mean()) - 1.0) < 0.02 and abs(float(norm.std()) - 0.1) < 0.02
    folder = write_model_folder(tmp_path / "m", TINY_B, 1)
    assert json.loads((folder / "config.json").read_text())["hidden_size"] == 192
    loaded = load_weights(folder, config, torch.float32, "cpu")
    assert all(torch.equal(loaded[k], one[k]) for k in one)


def test_random_init_command_line(tmp_path):
    from shrike_b200.weights.random_init import main

    (tmp_path / "c.json").write_text(json.dumps(TINY_A))
    main(["--config", str(tmp_path / "c.json"), "--seed", "3", "--out", str(tmp_path / "out")])
    assert (tmp_path / "out" / "model.safetensors").is_file()
    assert "lm_head.weight" not in SafetensorsFile(tmp_path / "out" / "model.safetensors").names()
