"""Trace replay: feed given token ids through the model step by step and write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

reads one JSON object per line from standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

runs the entries of a step as ONE batch through the engine's own step function (the model,
cache manager and kernels that generation uses; nothing is sampled), writes `<out>/<step>.f32`
(little-endian float32 [wanted, vocab], in the order of the entries and of `want`) when anything
is wanted, gives back what the requests named in `end` hold, and prints `done <step>`.
`--cuda-graphs` lets steps of single tokens replay captured graphs (padded to a bucket of
requests), the way the serving engine runs them.
`--max-tokens` sizes the page pool: the most tokens that live requests hold at any time, each
request's count rounded up to a multiple of 64; pages are reused as requests end.

The reference's `layover.replay` replays agent workloads over HTTP (layover/replay/__main__.py:43-77);
its nearest relative of this program is the chunked `prefill(..., all_logits=True)` loop of its
tests (tests/test_engine.py:47-59).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def parse_args(argv=None):
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at a time (each rounded up to 64)")
    parser.add_argument("--block-tokens", type=int, default=16, help="tokens per page (must divide 64)")
    parser.add_argument("--max-requests", type=int, default=16, help="most requests live at a time")
    parser.add_argument("--cuda-graphs", action="store_true",
                        help="replay steps of single tokens from captured CUDA graphs, as serving does")
    return parser.parse_args(argv)


def run(args, lines, say=print) -> int:
    import torch

    from .. import PagedKVCache, load_model
    from ..engine.batch import StepEntry
    from ..engine.step import StepFunction

    if 64 % args.block_tokens:
        raise SystemExit("--block-tokens must divide 64")
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    model = load_model(args.model, device="cuda", dtype=args.dtype)
    pages = max(1, -(-args.max_tokens // args.block_tokens))
    cache = PagedKVCache(model, pages, block_tokens=args.block_tokens, max_requests=args.max_requests)
    step_fn = StepFunction(model, cache, cuda_graphs=getattr(args, "cuda_graphs", False))
    live = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            seq = live.get(item["id"])
            if seq is None:
                seq = live[item["id"]] = cache.open(str(item["id"]))
            entries.append(StepEntry(seq, [int(t) for t in item["tokens"]], [int(w) for w in item.get("want", [])]))
        if entries:
            logits = step_fn(entries)
            if logits.shape[0]:
                host = logits.to(dtype=torch.float32, device="cpu").contiguous().numpy()
                host.astype("<f4", copy=False).tofile(out / f"{step}.f32")
        for name in record.get("end", []):
            seq = live.pop(name, None)
            if seq is not None:
                cache.close(seq)
        say(f"done {step}", flush=True)
    torch.cuda.synchronize()
    return 0


def main(argv=None) -> int:
    args = parse_args(argv)
    return run(args, sys.stdin)


if __name__ == "__main__":
    sys.exit(main())
