"""Decode and prefill throughput of the engine on one B200, Qwen3-4B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step. The default run is the 4B shape in bfloat16 at batch 8 over the
2,048 -> 4,096-token decode phase: the K timed steps are centred on a context of 3,072 tokens,
the mean of that phase. One JSON line on standard output:

  value      decoded tokens a second, K steps timed on the device with CUDA events
  e2e        the same through `layover_b200.Engine` (scheduler and sampler): host token ids in,
             host token ids out, every step
  prefill    one portion of 2,048 tokens from an empty cache; frac = flops / time / the bf16 peak
  roofline   bytes a decode step must read (every weight once + the live requests' K and V)
             / its time, against the measured copy bandwidth
  points     decode tokens a second at batch 1 and 64

Peaks come from MEASURED_PEAKS.json beside this file when it exists (else 6.65 TB/s and
1.59 PFLOP/s, an earlier measurement of the same kind of GPU). Inputs are synthetic token ids;
weights are seeded random values of the named shape. Weights (8 GB) are larger than the L2, so
nothing is flushed between steps.

`--impl reference` runs the unmodified CarlGergi/Layover installed under baseline/_ref through
its own Engine for the same metric, or prints why it cannot.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT, CONTEXT, PREFILL_TOKENS, PAGE = 2048, 4096, 2048, 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            found = {k: float(raw[k]) for k in FALLBACK_PEAKS if k in raw}
            if "hbm_gbs" in found and "bf16_tflops" in found:
                return {**FALLBACK_PEAKS, **found}, "measured"
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index, self.rows, self.process = index, [], None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.process is not None:
            time.sleep(0.25)
            self.process.terminate()
            self.thread.join(timeout=2)
        return False

    def summary(self) -> dict:
        clocks = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        maxima = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": reasons, "samples": len(clocks)}


# --------------------------------------------------------------------------------------- ours
def fill_requests(step_fn, cache, batch: int, tokens_each: int, vocab: int, gen):
    """Open `batch` requests and run `tokens_each` prompt tokens of each through the engine."""
    import torch
    from layover_b200 import StepEntry

    seqs = [cache.open(f"bench{i}") for i in range(batch)]
    for seq in seqs:
        at = 0
        while at < tokens_each:
            count = min(PREFILL_TOKENS, tokens_each - at)
            ids = torch.randint(0, vocab, (count,), generator=gen).tolist()
            step_fn([StepEntry(seq, ids, [])])
            at += count
    return seqs


def decode_point(model, batch: int, steps: int, warmup: int, gen, clocks=None) -> dict:
    """K decode steps of `batch` requests, timed on the device, centred on the middle of the decode phase."""
    import torch
    import layover_b200 as lb
    from layover_b200 import ops
    from layover_b200.engine.step import StepFunction

    vocab = model.spec.vocab_size
    start = max(1, (PROMPT + CONTEXT) // 2 - steps // 2 - warmup)
    pages = batch * (-(-(start + warmup + steps + 1) // PAGE))
    cache = lb.PagedKVCache(model, pages, block_tokens=PAGE, max_requests=batch)
    step_fn = StepFunction(model, cache, cuda_graphs=True, graph_sizes=(batch,), graph_max_tokens=CONTEXT)
    seqs = fill_requests(step_fn, cache, batch, start, vocab, gen)
    tokens = torch.randint(0, vocab, (warmup + steps, batch), generator=gen).tolist()
    for i in range(warmup):
        step_fn([lb.StepEntry(s, [tokens[i][j]], [0]) for j, s in enumerate(seqs)])
    torch.cuda.synchronize()
    launches_before = step_fn.replayed_launches + ops.LAUNCHES
    first_ctx = seqs[0].num_tokens
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if clocks is not None:
        clocks.__enter__()
    begin.record()
    for i in range(warmup, warmup + steps):
        step_fn([lb.StepEntry(s, [tokens[i][j]], [0]) for j, s in enumerate(seqs)])
    end.record()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.__exit__()
    ms = begin.elapsed_time(end) / steps
    mean_ctx = first_ctx + (steps + 1) / 2
    kv_bytes = batch * mean_ctx * sum(2 * n.kv_heads * n.head_dim for _, n, r in model.cache_needs() if r is None) * 2
    result = {"tok_s": batch * 1000.0 / ms, "ms_per_step": ms, "bytes": model.weight_bytes() + kv_bytes,
              "launches": step_fn.replayed_launches + ops.LAUNCHES - launches_before, "mean_ctx": mean_ctx,
              "graph_replays": step_fn.graph_replays}
    for seq in seqs:
        cache.close(seq)
    del cache, step_fn
    torch.cuda.empty_cache()
    return result


def prefill_point(model, gen, repeats: int = 5) -> dict:
    import torch
    import layover_b200 as lb
    from layover_b200.engine.step import StepFunction

    cache = lb.PagedKVCache(model, PREFILL_TOKENS // PAGE + 1, block_tokens=PAGE, max_requests=2)
    step_fn = StepFunction(model, cache)
    ids = torch.randint(0, model.spec.vocab_size, (PREFILL_TOKENS,), generator=gen).tolist()
    times = []
    for i in range(repeats + 2):
        seq = cache.open("p")
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        step_fn([lb.StepEntry(seq, ids, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(begin.elapsed_time(end))
        cache.close(seq)
    ms = statistics.median(times)
    return {"ms": ms, "tok_s": PREFILL_TOKENS * 1000.0 / ms}


def prefill_flops(cfg, layers: int, tokens: int) -> float:
    d, nq, nkv, h, inter = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.hidden_size, cfg.intermediate_size
    linear = 2.0 * tokens * layers * (h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * inter)
    attention = layers * 4.0 * nq * d * tokens * (tokens + 1) / 2
    return linear + attention + 2.0 * h * cfg.vocab_size


def e2e_point(model, batch: int, steps: int, warmup: int, gen) -> dict:
    """Through the public entry point: requests with host token ids, tokens read back every step
    (pipelined stepping: each call launches a step and takes in the tokens of the one before)."""
    import torch
    import layover_b200 as lb

    vocab = model.spec.vocab_size
    start = max(1, (PROMPT + CONTEXT) // 2 - steps // 2 - warmup)
    # requests that finish their prompt early decode while the others still prefill: leave room for
    # those tokens, so that every request is still running at the end of the timed steps
    slack = batch * (-(-start // PREFILL_TOKENS)) + 8
    budget = warmup + steps + slack
    pages = batch * (-(-(start + budget + 1) // PAGE))
    cache = lb.PagedKVCache(model, pages, block_tokens=PAGE, max_requests=batch)
    engine = lb.Engine(model, cache, lb.EngineConfig(batch, PREFILL_TOKENS, PREFILL_TOKENS), cuda_graphs=True)
    engine.step_fn.graph_sizes = (batch,)
    engine.step_fn.graph_table_width = cache.blocks_for(CONTEXT)
    for i in range(batch):
        prompt = torch.randint(0, vocab, (start,), generator=gen).tolist()
        engine.add_request(lb.Request(str(i), prompt, budget))
    while any(r.state is not lb.State.DECODE for r in engine.running) or engine.waiting:
        engine.step()
    for _ in range(warmup):
        engine.step_pipelined()
    torch.cuda.synchronize()
    produced = sum(len(r.generated) for r in engine.running)
    began = time.perf_counter()
    for _ in range(steps):
        engine.step_pipelined()      # launches one step and reads the tokens of the one before it
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - began
    if len(engine.running) != batch:
        raise RuntimeError("a request finished inside the timed steps: the end-to-end number would be wrong")
    produced = sum(len(r.generated) for r in engine.running) - produced
    width = engine.step_fn.graph_table_width
    h2d = 4 * lb.engine.BatchBuilder.buffer_size(lb.engine.BatchCapacity(batch, width), len(cache.paged), model.tile_sizes())
    return {"value": produced / elapsed, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch,
            "ms_per_step": 1000.0 * elapsed / steps}


def graph_time(fn, calls: int, reps: int = 10) -> float:
    """Milliseconds per call of `fn(i)`, `calls` of them captured in one CUDA graph and replayed
    `reps` times: device time of kernels running back to back, without host launch cost."""
    import torch

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(calls):
            fn(i)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(calls):
            fn(i)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(reps):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / reps / calls


def kernel_points(args) -> dict:
    """The dominant kernels alone at the benchmark's shapes, each over rotating operands larger than
    the L2: the four products of a layer at 8 and 2,048 tokens (with torch.mm, i.e. cuBLAS, beside
    them for scale) and the decode attention at batch 1, 8 and 64."""
    import math
    import torch
    import layover_b200 as lb
    from layover_b200 import ops

    cfg = lb.preset(args.model)
    d, nq, nkv, h, inter = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.hidden_size, cfg.intermediate_size
    shapes = {"qkv": ((nq + 2 * nkv) * d, h), "o": (h, nq * d), "gate_up": (2 * inter, h), "down": (h, inter)}
    ops.gemm_scratch("cuda"); ops.attention_scratch("cuda")
    out = {"gemm": {}, "attention_decode": {}}
    for tokens in (8, PREFILL_TOKENS):
        for name, (n, k) in shapes.items():
            copies = 24 if tokens <= 128 else 4
            weights = [(torch.randn(n, k, device="cuda") / math.sqrt(k)).to(torch.bfloat16) for _ in range(copies)]
            a = torch.randn(tokens, k, device="cuda").to(torch.bfloat16)
            c = torch.empty(tokens, n, device="cuda", dtype=torch.bfloat16)
            ours = graph_time(lambda i: ops.gemm_tcgen05(a, weights[i % copies], c), copies)
            lib = graph_time(lambda i: torch.mm(a, weights[i % copies].T, out=c), copies)
            out["gemm"][f"{name}_m{tokens}"] = {
                "us": round(ours * 1e3, 1), "cublas_us": round(lib * 1e3, 1),
                "tb_s": round(n * k * 2 / ours / 1e9, 2), "tflops": round(2.0 * tokens * n * k / ours / 1e9, 0)}
            del weights
    page, ctx = PAGE, (PROMPT + CONTEXT) // 2
    for batch in (1, 8, 64):
        pages_per = -(-ctx // page)
        layers = max(2, min(12, int(2e9 // (batch * pages_per * page * nkv * d * 4))))
        pools = torch.randn(layers, 2, batch * pages_per + 1, nkv, page, d, device="cuda").to(torch.bfloat16)
        table = torch.randperm(batch * pages_per, device="cuda").to(torch.int32).view(batch, pages_per)
        q = torch.randn(batch, nq * d, device="cuda").to(torch.bfloat16)
        o = torch.empty_like(q)
        cu = torch.arange(batch + 1, dtype=torch.int32, device="cuda")
        lens = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
        splits = ops.decode_splits(batch, nq, nkv, d, ctx, torch.cuda.get_device_properties(0).multi_processor_count)
        t = graph_time(lambda i: ops.attention_decode_bf16(q, pools[i % layers, 0], pools[i % layers, 1], o, table, cu, lens,
                                                           None, batch, nq, nkv, d, page, 1 / math.sqrt(d), 0, splits), layers)
        out["attention_decode"][f"b{batch}_ctx{ctx}"] = {
            "us": round(t * 1e3, 1), "splits": splits, "tb_s": round(batch * ctx * nkv * d * 4 / t / 1e9, 2)}
        del pools
    # one prompt of 2,048 tokens through the prompt-portion attention (tcgen05 where it takes the sizes)
    tokens = PREFILL_TOKENS
    if ops.attention_tcgen05_supports(nq, nkv, d, page):
        n_pages = -(-tokens // page)
        layers = 4
        pools = torch.randn(layers, 2, n_pages + 1, nkv, page, d, device="cuda").to(torch.bfloat16)
        table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(1, n_pages)
        q = torch.randn(tokens, nq * d, device="cuda").to(torch.bfloat16)
        o = torch.empty_like(q)
        cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
        lens = torch.tensor([tokens], dtype=torch.int32, device="cuda")
        n_tiles = -(-tokens // ops.TCGEN05_TILE)
        tile_seq = torch.zeros(n_tiles, dtype=torch.int32, device="cuda")
        tile_q0 = torch.arange(n_tiles, dtype=torch.int32, device="cuda") * ops.TCGEN05_TILE
        t = graph_time(lambda i: ops.attention_tcgen05_prefill(q, pools, i % layers, o, table, cu, lens, tile_seq, tile_q0,
                                                               n_tiles, nq, nkv, d, page, 1 / math.sqrt(d), 0), layers)
        flops = 4.0 * nq * d * tokens * (tokens + ops.TCGEN05_TILE) / 2      # both products, causal tiles
        out["attention_prefill"] = {f"t{tokens}": {"us": round(t * 1e3, 1), "tflops": round(flops / t / 1e9, 0)}}
        del pools
    return {"only": "kernels", **out, "gemm_status": ops.gemm_status(), "attention_status": ops.attention_tcgen05_status()}


def run_ours(args) -> dict:
    import torch
    import layover_b200 as lb

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    if args.only == "kernels":
        return kernel_points(args)
    cfg = lb.preset(args.model)
    layers_full = cfg.num_hidden_layers
    if args.layers:
        cfg = cfg.replace(num_hidden_layers=args.layers)
    gen = torch.Generator().manual_seed(0)
    model = lb.random_model(cfg, seed=0, device="cuda", dtype=args.dtype, std=0.02)
    pk, pk_source = peaks()
    if args.only == "decode":
        point = decode_point(model, args.batch, args.steps, args.warmup, gen)
        return {"only": "decode", "batch": args.batch, "layers_run": cfg.num_hidden_layers,
                "tok_s": round(point["tok_s"], 1), "ms_per_step": round(point["ms_per_step"], 4)}
    if args.only == "prefill":
        point = prefill_point(model, gen, repeats=max(1, args.steps))
        return {"only": "prefill", "layers_run": cfg.num_hidden_layers, "tok_s": round(point["tok_s"], 1),
                "ms": round(point["ms"], 3)}
    clocks = ClockSampler()
    main = decode_point(model, args.batch, args.steps, args.warmup, gen, clocks)
    prefill = prefill_point(model, gen)
    points = {}
    for batch in (1, 64):
        points[f"decode_b{batch}"] = round(decode_point(model, batch, max(16, args.steps // 2), args.warmup, gen)["tok_s"], 1)
    e2e = e2e_point(model, args.batch, max(16, args.steps // 2), args.warmup, gen)
    achieved = main["bytes"] / (main["ms_per_step"] * 1e-3) / 1e9
    flops = prefill_flops(cfg, cfg.num_hidden_layers, PREFILL_TOKENS)
    tflops_peak = pk["bf16_tflops"] if args.dtype == "bf16" else 75.0
    return {
        "metric": "decode tokens/s (Qwen3-4B shape, batch 8, context 2048->4096)", "value": round(main["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic token ids, seeded random weights", "impl": "ours",
        "config": {"model": args.model, "layers": layers_full, "layers_run": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
                   "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "tied_head": cfg.tie_word_embeddings,
                   "global_batch": args.batch, "prompt_len": PROMPT, "seq_len": CONTEXT, "timed_mean_context": round(main["mean_ctx"]),
                   "block_tokens": PAGE, "parallelism": "single GPU", "cuda_graphs": True,
                   "l2": "inputs larger than L2 (weights 8 GB), no flush", "peaks": pk_source},
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(prefill["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(prefill["ms"], 3),
                    "frac": round(flops / (prefill["ms"] * 1e-3) / (tflops_peak * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.summary(),
    }


# --------------------------------------------------------------------------------------- the reference
def run_reference(args) -> dict:
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "layover").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip --target install of the reference)"}
    sys.path.insert(0, str(ref))
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    try:
        import torch
        from layover.config import ModelConfig
        from layover.engine import Engine, EngineConfig, Request, State
        from layover.kv import PagedKVCache
        from layover.model import Qwen3
    except Exception as error:  # the reference or one of its imports is missing here
        return {"impl": "reference", "unavailable": f"import failed: {type(error).__name__}: {error}"[:200]}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    import layover_b200 as lb

    ours = lb.preset(args.model)
    cfg = ModelConfig.from_hf_dict(ours.to_hf_dict())
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = Qwen3(cfg).to(torch.bfloat16).eval()
    backend = "torch"
    try:
        from layover.kernels.triton_decode import paged_decode_attention_triton_trusted
        model.decode_attention = paged_decode_attention_triton_trusted
        backend = "triton"
    except Exception:
        pass
    batch, steps, warmup = args.batch, args.steps, args.warmup
    start = max(1, (PROMPT + CONTEXT) // 2 - steps // 2 - warmup)
    slack = batch * (-(-start // PREFILL_TOKENS)) + 8      # tokens decoded while other prompts still prefill
    blocks = batch * (-(-(start + warmup + steps + slack + 2) // PAGE)) + 2
    cache = PagedKVCache(cfg, blocks, "cuda", torch.bfloat16, PAGE)
    graphs = False
    if backend == "triton" and batch <= 8:
        try:
            from layover.decode_graphs import DecodeGraphs
            model.decode_graphs = DecodeGraphs(model, cache, max_tokens=CONTEXT)
            graphs = True
        except Exception:
            model.decode_graphs = None
    engine = Engine(model, cache, EngineConfig(batch, PREFILL_TOKENS, PREFILL_TOKENS))
    gen = torch.Generator().manual_seed(0)
    for i in range(batch):
        engine.add_request(Request(str(i), torch.randint(0, cfg.vocab_size, (start,), generator=gen).tolist(),
                                   warmup + steps + slack))
    clocks = ClockSampler()
    try:
        while engine.waiting or any(r.state is not State.DECODE for r in engine.running):
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        produced = sum(len(r.generated) for r in engine.running)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with clocks:
            began = time.perf_counter()
            begin.record()
            for _ in range(steps):
                engine.step()
            end.record()
            torch.cuda.synchronize()
            elapsed = time.perf_counter() - began
        produced = sum(len(r.generated) for r in engine.running + engine.finished) - produced
        device_ms = begin.elapsed_time(end) / steps
        # prefill of 2,048 tokens from an empty table
        from layover.kv import BlockTable
        pcache = PagedKVCache(cfg, PREFILL_TOKENS // PAGE + 1, "cuda", torch.bfloat16, PAGE)
        ids = torch.randint(0, cfg.vocab_size, (PREFILL_TOKENS,), generator=gen).cuda()
        times = []
        for i in range(5):
            table = BlockTable()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            model.prefill(pcache, table, ids, 0)
            torch.cuda.synchronize()
            times.append((time.perf_counter() - t0) * 1e3)
            pcache.release(table)
        prefill_ms = statistics.median(times[1:])
    except Exception as error:
        return {"impl": "reference", "unavailable": f"the reference failed on this GPU: {type(error).__name__}: {error}"[:240]}
    return {
        "metric": "decode tokens/s (Qwen3-4B shape, batch 8, context 2048->4096)", "value": round(batch * 1000.0 / device_ms, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(device_ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, torch default random weights", "impl": "reference",
        "config": {"model": args.model, "layers": cfg.num_hidden_layers, "layers_run": cfg.num_hidden_layers,
                   "global_batch": batch, "prompt_len": PROMPT, "seq_len": CONTEXT, "block_tokens": PAGE,
                   "decode_backend": backend, "cuda_graphs": graphs, "parallelism": "single GPU"},
        "e2e": {"value": round(produced / elapsed, 2), "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": 8 * batch},
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3)},
        "clocks": clocks.summary(),
    }


def main(argv=None) -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--model", default="qwen3-4b")
    parser.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="run fewer layers than the shape has (both numbers are reported)")
    parser.add_argument("--only", default="all", choices=["all", "decode", "prefill", "kernels"],
                        help="decode or prefill alone, as a small target for a profiler, or the dominant kernels "
                             "alone (prints a short line)")
    args = parser.parse_args(argv)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
