"""layover_b200: a small, whole LLM inference engine for one NVIDIA B200.

    from layover_b200 import load_model, PagedKVCache, Engine, EngineConfig, Request

    model = load_model("path/to/model", device="cuda", dtype="bf16")
    cache = PagedKVCache(model, num_blocks=4096, block_tokens=16)
    engine = Engine(model, cache, EngineConfig(max_batch=32, prefill_chunk=512, prefill_budget=512))
    engine.add_request(Request("a", prompt=[5, 17, 3], max_new_tokens=16))
    for request in engine.run_until_idle():
        print(request.request_id, request.generated)

The names follow CarlGergi/Layover's entry points (layover/weights.py:23, layover/kv/paged_cache.py:27,
layover/engine.py:64-99). Everything on the device runs in this package's own CUDA kernels for
sm_100a; there is no CPU path.
"""

from __future__ import annotations

import torch

from .cache import CacheManager, OutOfBlocks
from .config import Qwen3Config, load_config, preset, register_architecture, supported_architectures
from .engine import DEVICE_TOKEN, Engine, EngineConfig, Request, RequestTooLarge, State, StepEntry
from .models import load_model, random_model
from .parts.base import PagedKVNeed
from .sampling import SamplingParams
from .weights import write_model_folder

__version__ = "0.1.0"


def PagedKVCache(model, num_blocks: int, device=None, dtype=None, block_tokens: int = 16,
                 max_requests: int = 64) -> CacheManager:
    """The cache for `model`: `num_blocks` pages of `block_tokens` tokens for each group of layers
    with the same needs, plus `max_requests` slots of per-request state (the mixers' own and the
    record the sampler keeps). Device and dtype default to the model's (argument order of
    layover/kv/paged_cache.py:27-34)."""
    from . import ops

    device = model.device if device is None else device
    dtype = model.dtype if dtype is None else dtype
    return CacheManager(model.cache_needs(), num_blocks, block_tokens, dtype, device, max_requests, ops.RECORD_WORDS)


def blocks_for_pool(model, pool_gib: float, block_tokens: int = 16) -> int:
    """Pages that fit a pool of `pool_gib` GiB (layover/server.py:445-447)."""
    element = torch.empty((), dtype=model.dtype).element_size()
    bytes_per_token = sum(need.elements_per_token() * element for _, need, reads in model.cache_needs()
                          if reads is None and isinstance(need, PagedKVNeed))
    return max(1, int(pool_gib * 2**30 / (max(bytes_per_token, 1) * block_tokens)))


def generate(model, prompts: list[list[int]], max_new_tokens: int = 16, temperature: float = 0.0, seed: int = 0,
             stop_tokens=frozenset(), num_blocks: int | None = None, block_tokens: int = 16,
             config: EngineConfig | None = None, cuda_graphs: bool = False) -> list[list[int]]:
    """Token ids in, token ids out: run the prompts through a fresh cache and engine."""
    config = config or EngineConfig()
    if num_blocks is None:
        per_request = [-(-(len(p) + max_new_tokens) // block_tokens) for p in prompts]
        num_blocks = max(1, sum(sorted(per_request, reverse=True)[: config.max_batch]))
    cache = PagedKVCache(model, num_blocks, block_tokens=block_tokens,
                         max_requests=max(config.max_batch, 1))
    engine = Engine(model, cache, config, cuda_graphs=cuda_graphs)
    for index, prompt in enumerate(prompts):
        engine.add_request(Request(str(index), list(prompt), max_new_tokens, frozenset(stop_tokens),
                                   temperature, seed + index))
    done = {r.request_id: r.generated for r in engine.run_until_idle()}
    return [done[str(index)] for index in range(len(prompts))]


__all__ = [
    "CacheManager", "OutOfBlocks", "Qwen3Config", "load_config", "preset", "register_architecture",
    "supported_architectures", "DEVICE_TOKEN", "Engine", "EngineConfig", "Request", "RequestTooLarge", "State", "StepEntry",
    "load_model", "random_model", "SamplingParams", "write_model_folder", "PagedKVCache", "blocks_for_pool",
    "generate",
]
