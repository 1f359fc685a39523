"""The plain implementation against outputs of CarlGergi/Layover's own model code, recorded by
tests/golden/make_golden.py on tiny random models, and against itself."""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from golden.make_golden import CONFIGS, golden_weights, kept_rows, unpack
from plain_qwen3 import (plain_attention, plain_forward, plain_generate, plain_philox4x32, plain_rmsnorm,
                         plain_rope_tables, plain_sample, plain_uniform)

GOLDEN = json.loads((Path(__file__).parent / "golden" / "qwen3_golden.json").read_text())


@pytest.mark.parametrize("name", ["a", "b"])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_whole_prompts_match_the_reference(name, dtype_name):
    dtype = getattr(torch, dtype_name)
    record = GOLDEN[f"{name}/{dtype_name}"]
    weights = golden_weights(name)
    for prompt, packed in zip(record["prompts"], record["whole"]):
        expected = unpack(packed)
        got = plain_forward(CONFIGS[name], weights, prompt, dtype)[kept_rows(len(prompt))]
        eps = 2.0 ** -7 if dtype == torch.bfloat16 else 1e-5
        assert (got - expected).abs().max() <= 4 * eps * expected.abs().max()


@pytest.mark.parametrize("name", ["a", "b"])
def test_decode_rows_match_the_reference(name):
    record = GOLDEN[f"{name}/float32"]
    weights = golden_weights(name)
    for prompt, decode in zip(record["prompts"], record["decode"]):
        expected = unpack(decode["logits"])
        got = plain_forward(CONFIGS[name], weights, prompt + decode["tokens"], torch.float32)[len(prompt):]
        assert (got - expected).abs().max() <= 4e-5 * expected.abs().max()


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_tokens_match_the_reference_engine(name):
    record = GOLDEN[f"{name}/float32"]
    weights = golden_weights(name)
    for prompt, expected in zip(record["prompts"], record["greedy"]):
        assert plain_generate(CONFIGS[name], weights, prompt, len(expected)) == expected


def test_rmsnorm_and_rope_formulas():
    x = torch.tensor([[3.0, 4.0]])
    out = plain_rmsnorm(x, torch.tensor([2.0, 0.5]), 0.0)
    assert torch.allclose(out, torch.tensor([[2 * 3 / 12.5 ** 0.5, 0.5 * 4 / 12.5 ** 0.5]]))
    cos, sin = plain_rope_tables(torch.tensor([0, 1]), 4, 100.0, torch.float32)
    assert torch.allclose(cos[0], torch.ones(4)) and torch.allclose(sin[0], torch.zeros(4))
    assert torch.allclose(cos[1], torch.tensor([np.cos(1.0), np.cos(0.1), np.cos(1.0), np.cos(0.1)], dtype=torch.float32))


def test_attention_mask_groups_and_window():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = plain_attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])  # first query sees one key
    windowed = plain_attention(q, k, v, window=1)
    assert torch.allclose(windowed[:, 0], v[:, 0]) and torch.allclose(windowed[:, 2], v[:, 1])
    assert torch.allclose(plain_attention(q, k, v, window=100), out)


def test_philox_known_answers():
    # Random123's known-answer vectors for philox4x32-10
    zero = plain_philox4x32(np.zeros((1, 4), dtype=np.uint32), (0, 0))[0]
    assert [int(v) for v in zero] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    ones = plain_philox4x32(np.full((1, 4), 0xFFFFFFFF, dtype=np.uint32), (0xFFFFFFFF, 0xFFFFFFFF))[0]
    assert [int(v) for v in ones] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]


def test_sampling_distribution_and_determinism():
    logits = np.log(np.array([0.5, 0.25, 0.125, 0.125], dtype=np.float32))
    draws = [plain_sample(logits, 1.0, seed=5, step=s) for s in range(4000)]
    freq = np.bincount(draws, minlength=4) / 4000
    assert np.abs(freq - np.array([0.5, 0.25, 0.125, 0.125])).max() < 0.03
    assert plain_sample(logits, 1.0, 5, 7) == plain_sample(logits, 1.0, 5, 7)
    assert plain_sample(np.array([1.0, 3.0, 3.0]), 0.0, 0, 0) == 1
    u = plain_uniform(3, 9, 1000)
    assert u.min() > 0 and u.max() < 1
