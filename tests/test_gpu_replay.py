"""Replay on the GPU: the same requests whole, with the last 32 tokens decoded one by one, in
portions of changing size, and mixed with other requests on so few pages that they are used
again, in 32-bit and in bfloat16, all compared with the plain implementation."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import ROOT, TINY, TINY_PAGE, random_prompt, tolerance
from plain_qwen3 import plain_forward
from replay_helpers import max_live_tokens, mixed, portions, run_trace, tail_decoded, whole

pytestmark = pytest.mark.gpu

LENGTHS = {"a": [5, 17, 33, 70, 100, 41], "b": [1, 9, 64, 130, 77, 200], "c": [5, 140, 33, 300, 129, 260],
           "d": [1, 257, 64, 130, 77, 200]}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def requests_for(name):
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": random_prompt(vocab, n, seed=100 * ord(name) + i) for i, n in enumerate(LENGTHS[name])}


_expected = {}


def expected_rows(tiny_folders, name, dtype_name):
    key = (name, dtype_name)
    if key not in _expected:
        _, raw, weights = tiny_folders[name]
        _expected[key] = {rid: plain_forward(raw, weights, tokens, DTYPES[dtype_name]).numpy()
                          for rid, tokens in requests_for(name).items()}
    return _expected[key]


def compare(rows, expected, dtype):
    for rid, reference in expected.items():
        assert sorted(rows[rid]) == list(range(reference.shape[0])), f"{rid}: rows missing"
        got = np.stack([rows[rid][p] for p in range(reference.shape[0])])
        bound = tolerance(torch.from_numpy(reference), dtype)
        worst = np.abs(got - reference).max(axis=1)
        first_bad = np.nonzero(worst > bound)[0]
        assert first_bad.size == 0, (f"{rid}: first wrong position {first_bad[0]} of {reference.shape[0]}, "
                                     f"|diff| {worst[first_bad[0]]:.3e} > {bound:.3e}")


CUTS = {"whole": whole, "tail": tail_decoded, "portions": portions, "mixed": mixed}


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
@pytest.mark.parametrize("cut", list(CUTS))
def test_every_cut_matches_the_plain_implementation(tiny_folders, tmp_path, name, dtype_name, cut):
    folder, _, _ = tiny_folders[name]
    steps = CUTS[cut](requests_for(name))
    if cut == "mixed":
        # so few pages that a request which ends hands its pages to the next one
        assert max_live_tokens(steps) < sum(-(-n // 64) * 64 for n in LENGTHS[name])
        assert max(len(s["entries"]) for s in steps) == 4
        assert any(len(e["tokens"]) > 1 for s in steps for e in s["entries"] if len(s["entries"]) > 1)
    rows = run_trace(folder, dtype_name, steps, tmp_path, block_tokens=TINY_PAGE[name])
    compare(rows, expected_rows(tiny_folders, name, dtype_name), DTYPES[dtype_name])


@pytest.mark.parametrize("name", ["c", "d"])
@pytest.mark.parametrize("cut", list(CUTS))
def test_every_cut_at_the_served_head_size(tiny_folders, tmp_path, name, cut):
    """Head size 128 in bfloat16: prompt portions go through the tensor-core attention, with portions
    that start inside a tile of 128 keys and pages that are used again."""
    folder, _, _ = tiny_folders[name]
    requests = requests_for(name)
    # portions longer than a tile of 128 queries too, starting anywhere
    steps = portions(requests, sizes=(2, 150, 3, 131, 2, 33, 5, 1, 64, 2)) if cut == "portions" else CUTS[cut](requests)
    rows = run_trace(folder, "bfloat16", steps, tmp_path, block_tokens=TINY_PAGE[name])
    compare(rows, expected_rows(tiny_folders, name, "bfloat16"), torch.bfloat16)


SERVED_SHAPES = {   # (hidden, intermediate, query heads, KV heads) of the family's sizes, head size 128
    "0.6b": (1024, 3072, 16, 8), "4b": (2560, 9728, 32, 8), "14b": (5120, 17408, 40, 8), "32b": (5120, 25600, 64, 8),
}


@pytest.mark.parametrize("size", list(SERVED_SHAPES))
def test_one_layer_of_each_served_size(tmp_path, size):
    """The kernels at the family's real layer sizes (one layer, a small vocabulary): a prompt whole,
    its last tokens one by one, and two more requests decoding beside it, in bfloat16."""
    from safetensors.torch import load_file

    import layover_b200 as lb

    hidden, inter, q_heads, kv_heads = SERVED_SHAPES[size]
    config = lb.Qwen3Config(vocab_size=640, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=1,
                            num_attention_heads=q_heads, num_key_value_heads=kv_heads, head_dim=128,
                            max_position_embeddings=1024, rope_theta=1000000.0, rms_norm_eps=1e-6,
                            tie_word_embeddings=True)
    folder = tmp_path / "model"
    lb.write_model_folder(config, folder, seed=5, std=0.02, norm_std=0.1)
    raw = json.loads((folder / "config.json").read_text())
    weights = load_file(str(folder / "model.safetensors"))
    requests = {f"r{i}": random_prompt(640, n, seed=900 + i) for i, n in enumerate([150, 9, 40])}
    expected = {rid: plain_forward(raw, weights, tokens, torch.bfloat16).numpy() for rid, tokens in requests.items()}
    for cut in ("tail", "mixed"):
        rows = run_trace(folder, "bfloat16", CUTS[cut](requests), tmp_path / cut, block_tokens=16)
        compare(rows, expected, torch.bfloat16)


@pytest.mark.parametrize("name", ["a", "b"])
def test_32bit_logits_do_not_depend_on_the_cut_at_all(tiny_folders, tmp_path, name):
    """In the 32-bit path every sum has a fixed order, so cutting changes no bit."""
    folder, _, _ = tiny_folders[name]
    requests = requests_for(name)
    base = run_trace(folder, "float32", whole(requests), tmp_path / "whole", block_tokens=TINY_PAGE[name])
    for cut in ("tail", "portions", "mixed"):
        rows = run_trace(folder, "float32", CUTS[cut](requests), tmp_path / cut, block_tokens=TINY_PAGE[name])
        for rid in requests:
            for position, row in base[rid].items():
                assert np.array_equal(rows[rid][position], row), f"{cut}: {rid} position {position} differs"


def test_rows_that_are_not_wanted_are_not_written(tiny_folders, tmp_path):
    folder, raw, weights = tiny_folders["a"]
    tokens = random_prompt(256, 20, 5)
    steps = [
        {"step": 0, "entries": [{"id": "x", "tokens": tokens[:12], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "x", "tokens": tokens[12:], "want": [7, 0]}], "end": ["x"]},
    ]
    rows = run_trace(folder, "float32", steps, tmp_path, block_tokens=4)
    assert not (tmp_path / "0.f32").exists()
    data = np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(2, -1)
    reference = plain_forward(raw, weights, tokens).numpy()
    assert np.abs(data[0] - reference[19]).max() < 1e-4 and np.abs(data[1] - reference[12]).max() < 1e-4
    assert sorted(rows["x"]) == [12, 19]


def test_the_program_itself_step_by_step(tiny_folders, tmp_path):
    """bin/trace_run as a user runs it: a pipe in, `done <step>` after every step, files out."""
    folder, raw, weights = tiny_folders["b"]
    tokens = random_prompt(512, 40, 9)
    steps = portions({"p": tokens}, sizes=(16, 2, 22))
    env = {**os.environ, "PYTHONDONTWRITEBYTECODE": "1"}
    process = subprocess.Popen(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
         "--out", str(tmp_path), "--max-tokens", "64"],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    for step in steps:
        process.stdin.write(json.dumps(step) + "\n")
        process.stdin.flush()
        assert process.stdout.readline().strip() == f"done {step['step']}"
        wanted = sum(len(e["want"]) for e in step["entries"])
        assert (tmp_path / f"{step['step']}.f32").stat().st_size == wanted * 512 * 4   # written before `done`
    process.stdin.close()
    assert process.wait(timeout=120) == 0
    from replay_helpers import collect
    rows = collect(steps, tmp_path)
    reference = plain_forward(raw, weights, tokens).numpy()
    got = np.stack([rows["p"][i] for i in range(40)])
    assert np.abs(got - reference).max() <= tolerance(torch.from_numpy(reference), torch.float32)
