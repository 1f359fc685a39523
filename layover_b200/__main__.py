"""Command line: generate from token ids with a model folder or a named shape with random weights.

    python -m layover_b200 --model DIR --dtype bf16 --prompt-ids 5,17,3 --max-new-tokens 16
    python -m layover_b200 --preset tiny-b --random-weights --seed 1 --dtype fp32 --prompt-lens 9,64 --temperature 0.8

Option names and meanings follow the reference's server where it has them
(layover/server.py:415-434): --model, --device, --dtype {bf16,fp32}, --pool-gib, --block-tokens,
--max-batch, --prefill-chunk (also the per-step prompt budget, as server.py:461), --cuda-graphs.
--ignore-eos is the request option of that name (server.py:183,195). --max-batched-tokens is this
engine's own: one budget for a whole step, decoded tokens first. The HTTP server itself and the
agent options are not part of this engine. The result is one JSON object on standard output.
"""

from __future__ import annotations

import argparse
import json
import sys
import time


def parse_args(argv=None):
    p = argparse.ArgumentParser(prog="python -m layover_b200", description="Generate tokens on one B200")
    p.add_argument("--model", default=None, help="folder with config.json and *.safetensors")
    p.add_argument("--preset", default=None, help="a named shape instead of a folder (needs --random-weights)")
    p.add_argument("--random-weights", action="store_true", help="seeded random weights for --preset")
    p.add_argument("--seed", type=int, default=0, help="seed of the random weights and of sampling")
    p.add_argument("--device", default="cuda", choices=["cuda"], help="there is no CPU path")
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    p.add_argument("--pool-gib", type=float, default=2.0, help="KV pool size")
    p.add_argument("--num-blocks", type=int, default=None, help="KV pool size in pages (overrides --pool-gib)")
    p.add_argument("--block-tokens", type=int, default=16)
    p.add_argument("--max-batch", type=int, default=32)
    p.add_argument("--prefill-chunk", type=int, default=512)
    p.add_argument("--max-batched-tokens", type=int, default=None,
                   help="most tokens of a whole step, decoded tokens first (default: --prefill-chunk prompt tokens a "
                        "step, decoded tokens not counted)")
    p.add_argument("--ignore-eos", action="store_true", help="generate --max-new-tokens whatever is sampled")
    p.add_argument("--cuda-graphs", action="store_true", help="replay decode steps from CUDA graphs")
    p.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; may repeat")
    p.add_argument("--prompt-lens", default=None, help="comma-separated lengths of seeded random prompts")
    p.add_argument("--max-new-tokens", type=int, default=16)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--write-model", default=None, help="write the --preset's random model to this folder and exit")
    return p.parse_args(argv)


def main(argv=None) -> int:
    args = parse_args(argv)
    import torch

    import layover_b200 as lb

    if args.write_model:
        if not args.preset:
            raise SystemExit("--write-model needs --preset")
        lb.write_model_folder(lb.preset(args.preset), args.write_model, seed=args.seed)
        print(json.dumps({"wrote": args.write_model}))
        return 0
    if args.device == "cuda" and not torch.cuda.is_available():
        raise SystemExit("--device cuda requested but no CUDA GPU is available")
    if (args.model is None) == (args.preset is None):
        raise SystemExit("give exactly one of --model and --preset")
    if args.model:
        model = lb.load_model(args.model, device=args.device, dtype=args.dtype)
    else:
        if not args.random_weights:
            raise SystemExit("--preset has no weights of its own: add --random-weights")
        model = lb.random_model(lb.preset(args.preset), seed=args.seed, device=args.device, dtype=args.dtype)
    prompts = [[int(t) for t in text.split(",") if t] for text in args.prompt_ids]
    if args.prompt_lens:
        gen = torch.Generator().manual_seed(args.seed)
        for length in (int(n) for n in args.prompt_lens.split(",")):
            prompts.append(torch.randint(0, model.spec.vocab_size, (length,), generator=gen).tolist())
    if not prompts:
        raise SystemExit("no prompts: give --prompt-ids or --prompt-lens")
    blocks = args.num_blocks or lb.blocks_for_pool(model, args.pool_gib, args.block_tokens)
    cache = lb.PagedKVCache(model, blocks, block_tokens=args.block_tokens, max_requests=max(args.max_batch, 1))
    engine = lb.Engine(model, cache, lb.EngineConfig(args.max_batch, args.prefill_chunk, args.prefill_chunk,
                                                     args.max_batched_tokens), cuda_graphs=args.cuda_graphs)
    stop = frozenset() if getattr(model.cfg, "eos_token_id", None) is None else frozenset({model.cfg.eos_token_id})
    for index, prompt in enumerate(prompts):
        engine.add_request(lb.Request(str(index), prompt, args.max_new_tokens, stop, args.temperature, args.seed + index,
                                      ignore_eos=args.ignore_eos))
    began = time.perf_counter()
    finished = {r.request_id: r for r in engine.run_until_idle()}
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - began
    print(json.dumps({
        "generated": [finished[str(i)].generated for i in range(len(prompts))],
        "seconds": round(elapsed, 4),
        "stats": engine.stats,
        "pool_blocks": blocks,
    }))
    return 0


if __name__ == "__main__":
    sys.exit(main())
