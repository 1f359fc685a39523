"""Shared fixtures. Tests marked `gpu` need a CUDA device and are skipped without one; everything
else runs on the CPU. Model folders are made in temporary folders and never kept."""

from __future__ import annotations

import json
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for path in (str(ROOT), str(ROOT / "tests")):
    if path not in sys.path:
        sys.path.insert(0, path)

# Two tiny configurations that differ in every size and option the architecture has.
TINY = {
    "a": dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, max_position_embeddings=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True),
    "b": dict(vocab_size=512, hidden_size=96, intermediate_size=200, num_hidden_layers=3, num_attention_heads=6,
              num_key_value_heads=1, head_dim=32, max_position_embeddings=512, rope_theta=1000000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False),
}
# Two more with the head size of the served models, the only one the tensor-core attention takes:
# "c" has an even number of query heads per KV head (two heads per block) and is wide enough for the
# split products whose blocks form clusters (the fused q/k/v projection of decode steps); "d" has an
# odd number of heads per KV head and a narrow width.
TINY.update({
    "c": dict(vocab_size=384, hidden_size=512, intermediate_size=320, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=128, max_position_embeddings=512, rope_theta=1000000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=False),
    "d": dict(vocab_size=320, hidden_size=192, intermediate_size=256, num_hidden_layers=2, num_attention_heads=3,
              num_key_value_heads=1, head_dim=128, max_position_embeddings=512, rope_theta=10000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=True),
})
TINY_INIT = {"a": dict(std=0.02, norm_std=0.1), "b": dict(std=0.05, norm_std=0.2), "c": dict(std=0.04, norm_std=0.1),
             "d": dict(std=0.05, norm_std=0.2)}
TINY_PAGE = {"a": 4, "b": 16, "c": 16, "d": 8}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="needs a CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def tolerance(reference: torch.Tensor, dtype: torch.dtype) -> float:
    """The reference's own bound (tests/test_engine.py:41-44 there): 4 eps max|ref|, eps = 2^-7 for
    bfloat16 and 1e-5 for float32."""
    eps = 2.0 ** -7 if dtype == torch.bfloat16 else 1e-5
    return 4 * eps * reference.abs().max().item()


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """name -> (folder, raw config dict, weights by name as stored) for the tiny models."""
    from safetensors.torch import load_file

    import layover_b200 as lb

    out = {}
    for name, sizes in TINY.items():
        folder = tmp_path_factory.mktemp(f"tiny-{name}")
        lb.write_model_folder(lb.Qwen3Config(**sizes), folder, seed=11 + ord(name), **TINY_INIT[name])
        raw = json.loads((folder / "config.json").read_text())
        out[name] = (folder, raw, load_file(str(folder / "model.safetensors")))
    return out


def random_prompt(vocab: int, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=gen).tolist()
