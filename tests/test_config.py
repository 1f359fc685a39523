"""Configuration parsing, refusals, round trip and the architecture registry."""

import json

import pytest

import layover_b200 as lb
from layover_b200.config import (Qwen3Config, load_config, register_architecture, resolve_architecture,
                                 supported_architectures, unregister_architecture)
from conftest import TINY


def raw_b():
    return Qwen3Config(**TINY["b"]).to_hf_dict()


def test_round_trip_and_derived_sizes():
    cfg = Qwen3Config(**TINY["b"])
    again = Qwen3Config.from_hf_dict(cfg.to_hf_dict())
    assert again == cfg
    assert cfg.kv_groups == 6
    assert cfg.kv_bytes_per_token("bf16") == 3 * 2 * 1 * 32 * 2
    assert cfg.kv_bytes_per_token("fp32") == 2 * cfg.kv_bytes_per_token("bf16")


def test_defaults_follow_the_reference():
    raw = {"vocab_size": 10, "hidden_size": 32, "intermediate_size": 8, "num_hidden_layers": 1,
           "num_attention_heads": 4, "max_position_embeddings": 64}
    cfg = Qwen3Config.from_hf_dict(raw)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 8
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-6 and cfg.tie_word_embeddings is True
    assert Qwen3Config.from_hf_dict({**raw, "rope_parameters": {"rope_type": "default", "rope_theta": 5e5}}).rope_theta == 5e5
    assert Qwen3Config.from_hf_dict({**raw, "rope_theta": 7.0, "rope_scaling": {"rope_theta": 9.0}}).rope_theta == 7.0
    assert Qwen3Config.from_hf_dict({**raw, "eos_token_id": [7, 8]}).eos_token_id == 7
    assert Qwen3Config.from_hf_dict({**raw, "head_dim": 16}).head_dim == 16  # read, not derived


@pytest.mark.parametrize("change, message", [
    ({"model_type": "llama"}, "model_type"),
    ({"use_sliding_window": True}, "sliding-window"),
    ({"rope_scaling": {"type": "yarn"}}, "rope"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 4}, "divisible"),
    ({"head_dim": 7}, "even"),
    ({"num_hidden_layers": 0}, "positive"),
])
def test_refusals(change, message):
    with pytest.raises(ValueError, match=message):
        Qwen3Config.from_hf_dict({**raw_b(), **change})


def test_missing_keys_are_named():
    raw = raw_b()
    del raw["vocab_size"], raw["hidden_size"]
    with pytest.raises(ValueError, match="vocab_size.*hidden_size|hidden_size.*vocab_size"):
        Qwen3Config.from_hf_dict(raw)


def test_registry_resolves_by_architecture_then_model_type():
    assert "Qwen3ForCausalLM" in supported_architectures()
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).config_class is Qwen3Config
    assert resolve_architecture({"model_type": "qwen3"}).config_class is Qwen3Config
    with pytest.raises(ValueError, match="supported"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})


def test_registry_accepts_a_new_architecture(tmp_path):
    class ToyConfig:
        architecture, model_type = "ToyForCausalLM", "toy"

        @classmethod
        def from_hf_dict(cls, raw):
            return cls()

    register_architecture("ToyForCausalLM", "toy", ToyConfig, lambda cfg: None)
    try:
        (tmp_path / "config.json").write_text(json.dumps({"architectures": ["ToyForCausalLM"], "model_type": "toy"}))
        arch, cfg = load_config(tmp_path)
        assert arch.name == "ToyForCausalLM" and isinstance(cfg, ToyConfig)
    finally:
        unregister_architecture("ToyForCausalLM")
    assert "ToyForCausalLM" not in supported_architectures()


def test_presets_hold_the_benchmark_shapes():
    cfg = lb.preset("qwen3-4b")
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.head_dim, cfg.vocab_size) == (36, 2560, 128, 151936)
    assert lb.preset("tiny-a") == Qwen3Config(**TINY["a"])
    with pytest.raises(ValueError, match="unknown preset"):
        lb.preset("nope")


def test_model_spec_is_data():
    from layover_b200.models import spec_for_config

    spec = spec_for_config(Qwen3Config(**TINY["b"]))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    mixer = spec.layers[1].block.params["mixer"]
    assert mixer.kind == "attention" and mixer.params["kv_heads"] == 1 and mixer.params["head_dim"] == 32
    assert mixer.params["position"].params["theta"] == 1000000.0
    assert spec.head == "lm_head.weight"
    assert spec_for_config(Qwen3Config(**TINY["a"])).head is None
