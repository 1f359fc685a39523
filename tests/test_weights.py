"""The safetensors container, the loader's single error, and seeded random weights."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import layover_b200 as lb
from layover_b200.models import spec_for_config
from layover_b200.weights import (CheckpointMismatch, SafetensorsFile, TensorSpec, check_tensors, load_tensors,
                                  random_tensor, save_safetensors, write_model_folder)
from conftest import TINY


def test_container_round_trip_against_the_safetensors_package(tmp_path):
    tensors = {
        "a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
        "d": torch.arange(4, dtype=torch.int64), "e": torch.randn(2, 2).to(torch.float16),
    }
    save_safetensors(tensors, tmp_path / "ours.safetensors")
    theirs = load_file(str(tmp_path / "ours.safetensors"))          # their reader, our writer
    for name, t in tensors.items():
        assert theirs[name].dtype == t.dtype and torch.equal(theirs[name], t)
    save_file(tensors, str(tmp_path / "theirs.safetensors"))           # their writer, our reader
    handle = SafetensorsFile(tmp_path / "theirs.safetensors")
    assert sorted(handle.names()) == sorted(tensors)
    for name, t in tensors.items():
        got = handle.tensor(name)
        assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t)


def test_truncated_file_is_refused(tmp_path):
    path = tmp_path / "bad.safetensors"
    path.write_bytes(b"\xff" * 8 + b"{}")
    with pytest.raises(ValueError, match="header length"):
        SafetensorsFile(path)


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    specs = [TensorSpec("w1", (2, 3)), TensorSpec("w2", (4,), kind="vector"), TensorSpec("w3", (5, 5))]
    stored = {"w1": (3, 2), "w3": (5, 5), "extra.a": (1,), "extra.b": (2,)}
    with pytest.raises(CheckpointMismatch) as info:
        check_tensors(specs, stored)
    text = str(info.value)
    assert "missing (1): w2" in text
    assert "unexpected (2): extra.a, extra.b" in text
    assert "wrong shape (1): w1 expected [2, 3] got [3, 2]" in text
    assert info.value.missing == ["w2"] and info.value.unexpected == ["extra.a", "extra.b"]
    check_tensors(specs[2:], {"w3": (5, 5), "lm_head.weight": (1,)}, ignorable={"lm_head.weight"})


def test_folder_errors(tmp_path):
    with pytest.raises(FileNotFoundError, match="does not exist"):
        load_tensors(tmp_path / "nope", [], torch.float32, "cpu")
    with pytest.raises(FileNotFoundError, match="no safetensors"):
        load_tensors(tmp_path, [], torch.float32, "cpu")


def test_loaded_kinds_and_dtypes(tmp_path):
    save_safetensors({"m": torch.randn(4, 4), "v": torch.randn(4).to(torch.bfloat16), "k": torch.randn(2),
                      "t": torch.arange(3, dtype=torch.int64)}, tmp_path / "model.safetensors")
    specs = [TensorSpec("m", (4, 4)), TensorSpec("v", (4,), kind="vector"), TensorSpec("k", (2,), kind="keep32"),
             TensorSpec("t", (3,), kind="int")]
    got = load_tensors(tmp_path, specs, torch.bfloat16, "cpu")
    assert got["m"].dtype == torch.bfloat16          # a matrix takes the run's dtype
    assert got["v"].dtype == torch.float32           # norm weights are always 32-bit on the device
    assert got["k"].dtype == torch.float32           # stored in 32-bit, stays so
    assert got["t"].dtype == torch.int32             # integer tables as int32
    assert load_tensors(tmp_path, specs, torch.float32, "cpu")["m"].dtype == torch.float32
    with pytest.raises(CheckpointMismatch, match="integer table"):
        load_tensors(tmp_path, [TensorSpec("m", (4, 4), kind="int")], torch.float32, "cpu", ignorable={"v", "k", "t"})


def test_random_weights_are_seeded_by_name_not_by_order():
    a = random_tensor(TensorSpec("x.weight", (4, 4)), 3, 0.02, 0.0)
    b = random_tensor(TensorSpec("x.weight", (4, 4)), 3, 0.02, 0.0)
    c = random_tensor(TensorSpec("y.weight", (4, 4)), 3, 0.02, 0.0)
    d = random_tensor(TensorSpec("x.weight", (4, 4)), 4, 0.02, 0.0)
    assert torch.equal(a, b) and not torch.equal(a, c) and not torch.equal(a, d)
    n = random_tensor(TensorSpec("n", (1000,), kind="vector", init="ones"), 0, 0.02, 0.1)
    assert abs(n.mean().item() - 1.0) < 0.02 and 0.08 < n.std().item() < 0.12
    assert torch.equal(random_tensor(TensorSpec("n", (8,), kind="vector", init="ones"), 0, 0.02, 0.0), torch.ones(8))


@pytest.mark.parametrize("name", ["a", "b"])
def test_written_folder_has_the_checkpoint_names_and_reads_back(tmp_path, name):
    cfg = lb.Qwen3Config(**TINY[name])
    write_model_folder(cfg, tmp_path, seed=5, std=0.05, norm_std=0.2)
    raw = json.loads((tmp_path / "config.json").read_text())
    assert raw["architectures"] == ["Qwen3ForCausalLM"] and lb.Qwen3Config.from_hf_dict(raw) == cfg
    stored = load_file(str(tmp_path / "model.safetensors"))
    assert ("lm_head.weight" in stored) == (not cfg.tie_word_embeddings)
    assert stored["model.layers.0.self_attn.q_proj.weight"].shape == (cfg.num_attention_heads * cfg.head_dim, cfg.hidden_size)
    assert stored["model.layers.0.self_attn.k_norm.weight"].shape == (cfg.head_dim,)
    specs = spec_for_config(cfg).tensor_specs()
    assert sorted(s.name for s in specs) == sorted(stored)
    got = load_tensors(tmp_path, specs, torch.float32, "cpu")
    assert torch.equal(got["model.norm.weight"], stored["model.norm.weight"].float())
    # a second write with the same seed gives the same bytes
    other = tmp_path / "again"
    write_model_folder(cfg, other, seed=5, std=0.05, norm_std=0.2)
    assert (other / "model.safetensors").read_bytes() == (tmp_path / "model.safetensors").read_bytes()


def test_loading_a_folder_with_a_wrong_tensor_fails_before_any_device_work(tmp_path):
    cfg = lb.Qwen3Config(**TINY["a"])
    write_model_folder(cfg, tmp_path, seed=1)
    stored = load_file(str(tmp_path / "model.safetensors"))
    del stored["model.layers.1.mlp.up_proj.weight"]
    stored["model.layers.0.mlp.down_proj.weight"] = torch.zeros(3, 3)
    stored["stray"] = torch.zeros(1)
    save_file(stored, str(tmp_path / "model.safetensors"))
    specs = spec_for_config(cfg).tensor_specs()
    with pytest.raises(CheckpointMismatch) as info:
        load_tensors(tmp_path, specs, torch.float32, "cpu")
    assert info.value.missing == ["model.layers.1.mlp.up_proj.weight"]
    assert info.value.unexpected == ["stray"]
    assert info.value.wrong_shape[0][0] == "model.layers.0.mlp.down_proj.weight"


def test_no_cpu_path():
    from layover_b200.ops import KernelError

    with pytest.raises(KernelError, match="CUDA"):
        lb.random_model(lb.Qwen3Config(**TINY["a"]), device="cpu", dtype="fp32")
