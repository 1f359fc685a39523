"""Run CarlGergi/Layover's own model code on the CPU and record small outputs.

    python tests/golden/make_golden.py --reference PATH_TO_LAYOVER_CHECKOUT

The script builds two tiny random Qwen3 models from `golden_weights` below (a seeded
generator of this file, so the test can rebuild the same tensors without the reference),
loads them into the reference's `layover.model.Qwen3`, runs `prefill(..., all_logits=True)`
over a whole prompt and in chunks, a few batched `decode` steps and the reference engine's
greedy generation, and writes `tests/golden/qwen3_golden.json`. It also runs the plain
implementation of `tests/plain_qwen3.py` on the same inputs and prints the differences.

`tests/test_plain.py` reads the JSON and compares the plain implementation with it; the
reference itself is not needed for that.
"""

from __future__ import annotations

import argparse
import base64
import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent

CONFIGS = {
    "a": {
        "model_type": "qwen3", "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128,
        "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
        "max_position_embeddings": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
        "tie_word_embeddings": True,
    },
    "b": {
        "model_type": "qwen3", "vocab_size": 512, "hidden_size": 96, "intermediate_size": 200,
        "num_hidden_layers": 3, "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 32,
        "max_position_embeddings": 512, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
        "tie_word_embeddings": False,
    },
}
INIT = {"a": (0.02, 0.1), "b": (0.05, 0.2)}
PROMPT_LENGTHS = {"a": [5, 17, 33], "b": [1, 9, 64, 130]}


def tensor_shapes(raw: dict) -> dict[str, tuple[int, ...]]:
    hidden, inter, dim = raw["hidden_size"], raw["intermediate_size"], raw["head_dim"]
    nq, nkv = raw["num_attention_heads"], raw["num_key_value_heads"]
    shapes = {"model.embed_tokens.weight": (raw["vocab_size"], hidden), "model.norm.weight": (hidden,)}
    for i in range(raw["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shapes[p + "input_layernorm.weight"] = (hidden,)
        shapes[p + "post_attention_layernorm.weight"] = (hidden,)
        shapes[p + "self_attn.q_proj.weight"] = (nq * dim, hidden)
        shapes[p + "self_attn.k_proj.weight"] = (nkv * dim, hidden)
        shapes[p + "self_attn.v_proj.weight"] = (nkv * dim, hidden)
        shapes[p + "self_attn.o_proj.weight"] = (hidden, nq * dim)
        shapes[p + "self_attn.q_norm.weight"] = (dim,)
        shapes[p + "self_attn.k_norm.weight"] = (dim,)
        shapes[p + "mlp.gate_proj.weight"] = (inter, hidden)
        shapes[p + "mlp.up_proj.weight"] = (inter, hidden)
        shapes[p + "mlp.down_proj.weight"] = (hidden, inter)
    if not raw["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (raw["vocab_size"], hidden)
    return shapes


def golden_weights(name: str, seed: int = 1234) -> dict[str, torch.Tensor]:
    """Matrices ~ N(0, std), norm weights 1 + N(0, norm_std), drawn in sorted-name order."""
    std, norm_std = INIT[name]
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for tensor, shape in sorted(tensor_shapes(CONFIGS[name]).items()):
        noise = torch.randn(shape, generator=gen, dtype=torch.float32)
        out[tensor] = 1.0 + norm_std * noise if len(shape) == 1 else std * noise
    return out


def golden_prompts(name: str, seed: int = 99) -> list[list[int]]:
    gen = torch.Generator().manual_seed(seed)
    vocab = CONFIGS[name]["vocab_size"]
    return [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in PROMPT_LENGTHS[name]]


def pack(rows: torch.Tensor) -> dict:
    """Rows of 32-bit floats as base64 of their little-endian bytes, to keep the file small."""
    rows = rows.float().contiguous()
    return {"shape": list(rows.shape), "f32": base64.b64encode(rows.numpy().astype("<f4").tobytes()).decode()}


def unpack(packed: dict) -> torch.Tensor:
    import numpy as np

    flat = np.frombuffer(base64.b64decode(packed["f32"]), dtype="<f4").copy()
    return torch.from_numpy(flat).reshape(packed["shape"])


def kept_rows(count: int) -> list[int]:
    """The rows of a prompt whose logits are recorded: first, middle, last."""
    return sorted({0, count // 2, count - 1})


def run_reference(name: str, dtype: torch.dtype) -> dict:
    from layover.config import ModelConfig
    from layover.engine import Engine, EngineConfig, Request
    from layover.kv import BlockTable, PagedKVCache
    from layover.model import Qwen3

    cfg = ModelConfig.from_hf_dict(CONFIGS[name])
    model = Qwen3(cfg).to(dtype).eval()
    state = {k: v.to(dtype) for k, v in golden_weights(name).items()}
    # as layover/weights.py:36-44: a tied head is not in the checkpoint and aliases the embedding
    missing = model.load_state_dict(state, strict=False)
    assert not missing.unexpected_keys and set(missing.missing_keys) <= {"lm_head.weight"}
    if cfg.tie_word_embeddings:
        model.lm_head.weight = model.model.embed_tokens.weight
    record = {"prompts": golden_prompts(name), "whole": [], "chunked_max_diff": [], "decode": [], "greedy": []}
    for prompt in record["prompts"]:
        tokens = torch.tensor(prompt)
        cache, table = PagedKVCache(cfg, 64, dtype=dtype, block_tokens=4), BlockTable()
        whole = model.prefill(cache, table, tokens, 0, all_logits=True).float()
        record["whole"].append(pack(whole[kept_rows(len(prompt))]))
        cache, table = PagedKVCache(cfg, 64, dtype=dtype, block_tokens=4), BlockTable()
        parts = [model.prefill(cache, table, tokens[s : s + 7], s, all_logits=True) for s in range(0, len(prompt), 7)]
        record["chunked_max_diff"].append(float((torch.cat(parts).float() - whole).abs().max()))
        # four decode steps with given tokens, as the reference's own tests do (tests/test_engine.py:88-105)
        follow = [(3 * i + 1) % cfg.vocab_size for i in range(4)]
        rows = [model.decode(cache, [table], torch.tensor([token]))[0].float() for token in follow]
        record["decode"].append({"tokens": follow, "logits": pack(torch.stack(rows))})
    engine = Engine(model, PagedKVCache(cfg, 256, dtype=dtype, block_tokens=4), EngineConfig(8, 16, 32))
    for i, prompt in enumerate(record["prompts"]):
        engine.add_request(Request(str(i), prompt, 8))
    done = {r.request_id: r.generated for r in engine.run_until_idle()}
    record["greedy"] = [done[str(i)] for i in range(len(record["prompts"]))]
    return record


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="a checkout of CarlGergi/Layover")
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    sys.path.insert(0, str(HERE.parent))
    sys.dont_write_bytecode = True
    from plain_qwen3 import plain_forward

    out = {}
    for name in CONFIGS:
        for dtype_name, dtype in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            record = run_reference(name, dtype)
            worst = 0.0
            for prompt, whole in zip(record["prompts"], record["whole"]):
                ours = plain_forward(CONFIGS[name], golden_weights(name), prompt, dtype)[kept_rows(len(prompt))]
                ref = unpack(whole)
                worst = max(worst, float((ours - ref).abs().max()) / float(ref.abs().max()))
            print(f"{name} {dtype_name}: plain vs reference, worst |diff|/max|ref| = {worst:.3e}; "
                  f"reference chunked vs whole max diff = {max(record['chunked_max_diff']):.3e}")
            out[f"{name}/{dtype_name}"] = record
    (HERE / "qwen3_golden.json").write_text(json.dumps(out))
    print("wrote", HERE / "qwen3_golden.json")


if __name__ == "__main__":
    main()
