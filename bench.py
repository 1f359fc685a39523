"""Decode and prefill throughput of the engine on one B200, random weights of a named Qwen3 shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config 4b|4b-fp32|8b-mixed|32b-long]

A step is one decode step. Every run prints ONE JSON line on standard output.

--config 4b (the default, the headline): the 4B shape in bfloat16 at batch 8 over the
2,048 -> 4,096-token decode phase; the K timed steps are centred on a context of 3,072 tokens,
the mean of that phase.

  value      decoded tokens a second, K steps timed on the device with CUDA events; a step is what
             serving runs: the captured decode graph with the sampling kernel in it
  e2e        the same through `layover_b200.Engine` (scheduler and sampler): host token ids in,
             host token ids out, every step
  prefill    one portion of 2,048 tokens from an empty cache; frac = flops / time / the bf16 peak
  roofline   bytes a decode step must read (every weight once + the live requests' K and V)
             / its time, against the measured copy bandwidth
  points     decode tokens a second at batch 1 and 64
  contexts   milliseconds per step at batch 8 with the timed steps centred on 2,048 and 3,072 tokens of
             context and, for 4,096, ending there (the context is full then)
  kernels    the dominant kernels alone (the four products of a layer at 8 and at 2,048 tokens, the
             decode attention at batch 1, 8 and 64, the prompt attention): microseconds and the
             fraction of the measured peak (copy bandwidth for the decode kernels, the bf16 burst
             rate for the prompt kernels)

Before anything is timed, one decode step is run twice from the same state, replayed from its
captured graph and launch by launch, and the logits and tokens must agree bit for bit.

--config 4b-fp32: the same shape through the true 32-bit path (FFMA products): decode at batch 1
and 8 and the prefill. --config 8b-mixed: the 8B shape, 32 requests with prompts of 128..8,192
tokens (seeded), prompt portions of 2,048 tokens beside decoding requests, 512 new tokens each,
through `Engine`. --config 32b-long: the 32B shape, 8 prompts of 32,768 tokens, then 256 greedy
decode steps.

Peaks come from MEASURED_PEAKS.json beside this file when it exists (else 6.65 TB/s and
1.59 PFLOP/s, an earlier measurement of the same kind of GPU). Inputs are synthetic token ids;
weights are seeded random values of the named shape. Weights (8 GB and more) are larger than the
L2, so nothing is flushed between steps.

`--impl reference` runs the unmodified CarlGergi/Layover installed under baseline/_ref through
its own Engine for the headline metric, or prints why it cannot.
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
FP32_TFLOPS = 75.0       # nominal FFMA rate of the part; only the 32-bit path's prefill fraction uses it
CONFIGS = {"4b": ("qwen3-4b", "bf16"), "4b-fp32": ("qwen3-4b", "fp32"), "8b-mixed": ("qwen3-8b", "bf16"),
           "32b-long": ("qwen3-32b", "bf16")}
METRIC = "decode tokens/s (Qwen3-4B shape, batch 8, context 2048->4096)"


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


def config_record(cfg, model_name: str, layers_run: int, batch: int, prompt: int, seq_len: int, mean_ctx: float,
                  graphs: bool, pk_source: str) -> dict:
    """The `config` of a line: every size of the layers, flat. Both arms print the same keys."""
    return {"model": model_name, "layers": cfg.num_hidden_layers, "layers_run": layers_run, "hidden": cfg.hidden_size,
            "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "tied_head": cfg.tie_word_embeddings,
            "global_batch": batch, "prompt_len": prompt, "seq_len": seq_len, "timed_mean_context": round(mean_ctx),
            "block_tokens": PAGE, "parallelism": "single GPU", "cuda_graphs": graphs,
            "l2": "inputs larger than L2 (weights of 8 GB or more), no flush", "peaks": pk_source}


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


def kv_bytes_per_token(model) -> int:
    from layover_b200.parts.base import PagedKVNeed

    element = 2 if str(model.dtype).endswith("bfloat16") else 4
    return sum(need.elements_per_token() * element for _, need, reads in model.cache_needs()
               if reads is None and isinstance(need, PagedKVNeed))


def check_graph_replay(model, gen) -> None:
    """One decode step, replayed from its captured graph and run launch by launch from the same
    state (two caches filled alike): logits and sampled tokens must agree bit for bit."""
    import torch
    import layover_b200 as lb
    from layover_b200.engine.step import StepFunction

    vocab, batch, outputs = model.spec.vocab_size, 5, []         # 5 rows in a bucket of 8: padded rows run too
    prompts = [torch.randint(0, vocab, (40 + 300 * i,), generator=gen).tolist() for i in range(batch)]
    for replay in (True, False):
        cache = lb.PagedKVCache(model, batch * 100, block_tokens=PAGE, max_requests=8)
        step_fn = StepFunction(model, cache, cuda_graphs=True, graph_max_tokens=CONTEXT)
        step_fn.replay_graphs = replay
        seqs = [cache.open(f"check{i}") for i in range(batch)]
        for seq, prompt in zip(seqs, prompts):
            step_fn([lb.StepEntry(seq, prompt, [])])
        logits = step_fn([lb.StepEntry(seq, [17 + i], [0]) for i, seq in enumerate(seqs)]).clone()
        tokens = step_fn.sample([lb.StepEntry(seq, [lb.DEVICE_TOKEN], [0]) for seq in seqs]).result()
        outputs.append((logits.cpu(), tokens))
        if replay and step_fn.graph_replays != 2:
            raise RuntimeError("bench.py: the decode steps of the check did not replay a graph")
        for seq in seqs:
            cache.close(seq)
        del cache, step_fn
    (graph_logits, graph_tokens), (eager_logits, eager_tokens) = outputs
    if not torch.equal(graph_logits, eager_logits) or graph_tokens != eager_tokens:
        worst = (graph_logits - eager_logits).abs().max().item()
        raise RuntimeError(f"bench.py: a replayed decode step differs from the same step without a graph "
                           f"(largest |difference| of logits {worst:.3e}): nothing was timed")
    if not torch.isfinite(graph_logits).all():
        raise RuntimeError("bench.py: the checked decode step has logits that are not finite")
    torch.cuda.empty_cache()


def decode_point(model, batch: int, steps: int, warmup: int, gen, clocks=None, centre: int | None = None,
                 first_ctx: int | None = None, graph_tokens: int = CONTEXT) -> dict:
    """K decode steps of `batch` requests, timed on the device, centred on the context `centre` (or
    starting at `first_ctx`). A step is `StepFunction.sample` on the tokens the step before sampled:
    the captured graph (with the sampling kernel), one copy in and one copy out."""
    import torch
    import layover_b200 as lb
    from layover_b200 import ops
    from layover_b200.engine.step import StepFunction

    vocab = model.spec.vocab_size
    if first_ctx is None:
        centre = (PROMPT + CONTEXT) // 2 if centre is None else centre
        first_ctx = max(1, centre - steps // 2 - warmup)
    pages = batch * (-(-(first_ctx + warmup + steps + 1) // PAGE))
    cache = lb.PagedKVCache(model, pages, block_tokens=PAGE, max_requests=batch)
    step_fn = StepFunction(model, cache, cuda_graphs=True, graph_sizes=(batch,), graph_max_tokens=graph_tokens)
    seqs = fill_requests(step_fn, cache, batch, first_ctx - 1, vocab, gen)
    # every graph the timed steps replay is captured now, not inside the timed region
    step_fn.capture_all(tokens=first_ctx + warmup + steps + 1, from_tokens=first_ctx)
    first = torch.randint(0, vocab, (batch,), generator=gen).tolist()
    pending = step_fn.sample([lb.StepEntry(s, [first[j]], [0]) for j, s in enumerate(seqs)])   # now every record has a token
    entries = lambda: [lb.StepEntry(s, [lb.DEVICE_TOKEN], [0]) for s in seqs]
    for _ in range(warmup):
        pending.result()
        pending = step_fn.sample(entries())
    pending.result()
    torch.cuda.synchronize()
    launches_before = step_fn.replayed_launches + ops.LAUNCHES
    replays_before = step_fn.graph_replays
    start_ctx = seqs[0].num_tokens
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if clocks is not None:
        clocks.__enter__()
    begin.record()
    waiting = None
    for _ in range(steps):
        pending = step_fn.sample(entries())
        if waiting is not None:
            waiting.result()         # the host reads a step's tokens while the device runs the next
        waiting = pending
    end.record()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.__exit__()
    waiting.result()
    ms = begin.elapsed_time(end) / steps
    mean_ctx = start_ctx + (steps + 1) / 2
    kv_bytes = batch * mean_ctx * kv_bytes_per_token(model)
    result = {"tok_s": batch * 1000.0 / ms, "ms_per_step": ms, "bytes": model.weight_bytes() + kv_bytes,
              "launches": step_fn.replayed_launches + ops.LAUNCHES - launches_before, "mean_ctx": mean_ctx,
              "graph_replays": step_fn.graph_replays - replays_before}
    if result["graph_replays"] != steps:
        raise RuntimeError("bench.py: a timed decode step did not replay its graph")
    for seq in seqs:
        cache.close(seq)
    del cache, step_fn
    torch.cuda.empty_cache()
    return result


def prefill_point(model, gen, repeats: int = 5, graphs: bool = True) -> dict:
    """One prompt portion of PREFILL_TOKENS tokens, alone in its step, as the engine runs it: replayed
    from a captured graph (`graphs`), or launch by launch."""
    import torch
    import layover_b200 as lb
    from layover_b200.engine.step import StepFunction

    cache = lb.PagedKVCache(model, PREFILL_TOKENS // PAGE + 1, block_tokens=PAGE, max_requests=2)
    step_fn = StepFunction(model, cache, cuda_graphs=graphs, portion_graph_tokens=(PREFILL_TOKENS,))
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
    engine.step_fn.capture_all(tokens=start + budget, from_tokens=start)     # not inside the timed steps
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
    width = engine.step_fn.graph_width_for(cache.blocks_for(start + budget))
    h2d = 4 * lb.engine.BatchBuilder.buffer_size(lb.engine.BatchCapacity(batch, width), len(cache.paged), model.tile_sizes())
    d2h = 4 * (batch + engine.step_fn.sampler.n_status)
    return {"value": produced / elapsed, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
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


def kernel_points(model_name: str, pk: dict, with_library: bool) -> dict:
    """The dominant kernels alone at the benchmark's shapes, each over rotating operands larger than
    the L2: the four products of a layer at 8 and 2,048 tokens (with torch.mm, i.e. cuBLAS, beside
    them for scale when `with_library`), the decode attention at batch 1, 8 and 64 and the prompt
    attention. `frac` is of the measured peak: copy bandwidth for the few-token products and the
    decode attention, the bf16 burst rate for the 2,048-token products and the prompt attention."""
    import math
    import torch
    import layover_b200 as lb
    from layover_b200 import ops

    cfg = lb.preset(model_name)
    d, nq, nkv, h, inter = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.hidden_size, cfg.intermediate_size
    shapes = {"qkv": ((nq + 2 * nkv) * d, h), "o": (h, nq * d), "gate_up": (2 * inter, h), "down": (h, inter)}
    ops.gemm_scratch("cuda"); ops.attention_scratch("cuda")
    out = {}
    for tokens in (8, PREFILL_TOKENS):
        for name, (n, k) in shapes.items():
            copies = 24 if tokens <= 128 else 4
            weights = [(torch.randn(n, k, device="cuda") / math.sqrt(k)).to(torch.bfloat16) for _ in range(copies)]
            a = torch.randn(tokens, k, device="cuda").to(torch.bfloat16)
            c = torch.empty(tokens, n, device="cuda", dtype=torch.bfloat16)
            ours = graph_time(lambda i: ops.gemm_tcgen05(a, weights[i % copies], c), copies)
            row = {"us": round(ours * 1e3, 1)}
            if tokens <= 128:
                row["frac"] = round(n * k * 2 / (ours * 1e-3) / 1e9 / pk["hbm_gbs"], 3)
            else:
                row["frac"] = round(2.0 * tokens * n * k / (ours * 1e-3) / 1e12 / pk["bf16_tflops"], 3)
            if with_library:
                lib = graph_time(lambda i: torch.mm(a, weights[i % copies].T, out=c), copies)
                row["cublas_us"] = round(lib * 1e3, 1)
            out[f"{name}_m{tokens}"] = row
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
        splits, stages = ops.decode_plan(batch, nq, nkv, d, ctx, torch.cuda.get_device_properties(0).multi_processor_count)
        t = graph_time(lambda i: ops.attention_decode_bf16(q, pools[i % layers, 0], pools[i % layers, 1], o, table, cu, lens,
                                                           None, batch, nq, nkv, d, page, 1 / math.sqrt(d), 0, splits, stages),
                       layers)
        out[f"attn_decode_b{batch}"] = {"us": round(t * 1e3, 1), "splits": splits, "stages": stages,
                                        "frac": round(batch * ctx * nkv * d * 4 / (t * 1e-3) / 1e9 / pk["hbm_gbs"], 3)}
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
        out[f"attn_prefill_t{tokens}"] = {"us": round(t * 1e3, 1),
                                          "frac": round(flops / (t * 1e-3) / 1e12 / pk["bf16_tflops"], 3)}
        del pools
    if ops.gemm_status() or ops.attention_tcgen05_status():
        raise RuntimeError("bench.py: a tensor-core kernel reported a wait that ran out")
    torch.cuda.empty_cache()
    return out


def plan_points(model_name: str, pk: dict) -> dict:
    """The decode attention alone over launch plans (splits, K/V stages), for requests of equal length
    and for lengths spread evenly over 0.1..1 of the longest: microseconds of each plan, the plan that
    `ops.decode_plan` picks knowing only the longest (`equal`) and knowing the mean too (`chosen`), and
    the time the bytes would take at the measured copy bandwidth."""
    import math
    import torch
    import layover_b200 as lb
    from layover_b200 import ops

    cfg = lb.preset(model_name)
    d, nq, nkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ops.attention_scratch("cuda")
    gen = torch.Generator().manual_seed(1)
    plans = [(splits, stages) for stages in (3, 2) for splits in (1, 2, 4, 8)]
    out = {}
    for batch in (8, 16, 32, 64):
        for longest in (3072, 8192):
            for spread in ("equal", "uniform"):
                lengths = [longest] * batch
                if spread == "uniform":
                    lengths = (torch.rand(batch, generator=gen) * 0.9 * longest + 0.1 * longest).int().tolist()
                    lengths[0] = longest
                pages_per = -(-longest // PAGE)
                total_pages = sum(-(-n // PAGE) for n in lengths)
                layers = max(2, min(8, int(1.5e9 // (total_pages * PAGE * nkv * d * 4))))
                pools = torch.randn(layers, 2, total_pages + 1, nkv, PAGE, d, device="cuda").to(torch.bfloat16)
                table = torch.zeros(batch, pages_per, dtype=torch.int32)
                order, at = torch.randperm(total_pages, generator=gen).to(torch.int32), 0
                for i, n in enumerate(lengths):
                    count = -(-n // PAGE)
                    table[i, :count] = order[at:at + count]
                    at += count
                table = table.cuda()
                q = torch.randn(batch, nq * d, device="cuda").to(torch.bfloat16)
                o = torch.empty_like(q)
                cu = torch.arange(batch + 1, dtype=torch.int32, device="cuda")
                lens = torch.tensor(lengths, dtype=torch.int32, device="cuda")
                row = {}
                for splits, stages in plans:
                    t = graph_time(lambda i: ops.attention_decode_bf16(q, pools[i % layers, 0], pools[i % layers, 1], o, table, cu,
                                                                       lens, None, batch, nq, nkv, d, PAGE, 1 / math.sqrt(d), 0,
                                                                       splits, stages), layers)
                    row[f"{splits}x{stages}"] = round(t * 1e3, 1)
                mean = sum(lengths) // batch
                row["equal"] = "%dx%d" % ops.decode_plan(batch, nq, nkv, d, longest, sms)
                row["chosen"] = "%dx%d" % ops.decode_plan(batch, nq, nkv, d, longest, sms, mean)
                row["bytes_us"] = round(sum(lengths) * nkv * d * 4 / pk["hbm_gbs"] / 1e3, 1)
                out[f"b{batch}_{longest}_{spread}"] = row
                del pools
    torch.cuda.empty_cache()
    return out


def timeline_point(model, batch: int, gen) -> dict:
    """Where a replayed decode step's time goes, kernel by kernel: a torch.profiler trace of three
    replays at a context of 3,000 tokens; for one middle layer each kernel's own duration and the time
    from the end of the kernel before it to its own end (kernels overlap under programmatic dependent
    launch, so the second column is what a kernel adds to the step)."""
    import re
    import torch
    import layover_b200 as lb
    from layover_b200.engine.step import StepFunction
    from torch.profiler import ProfilerActivity, profile

    start = (PROMPT + CONTEXT) // 2 - 72
    cache = lb.PagedKVCache(model, batch * (-(-(start + 64) // PAGE)), block_tokens=PAGE, max_requests=batch)
    step_fn = StepFunction(model, cache, cuda_graphs=True, graph_sizes=(batch,), graph_max_tokens=CONTEXT)
    seqs = fill_requests(step_fn, cache, batch, start, model.spec.vocab_size, gen)
    entries = lambda: [lb.StepEntry(s, [5], [0]) for s in seqs]
    for _ in range(5):
        step_fn.sample(entries()).result()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step_fn.sample(entries()).result()
        torch.cuda.synchronize()
    events = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "memcpy" not in e.name.lower()]
    events.sort(key=lambda e: e.time_range.start)

    def short(name: str) -> str:
        found = re.search(r"(\w+_kernel)(<[^>]*>)?", name)
        return (found.group(1) + (found.group(2) or "")) if found else name[:60]

    kernels = [(short(e.name), e.time_range.start, e.time_range.end) for e in events]
    last = kernels[-(len(kernels) // 3):]
    attention = [i for i, k in enumerate(last) if "attention_decode" in k[0]]
    per_layer = attention[1] - attention[0]
    middle = attention[len(attention) // 2]
    rows, previous_end = [], last[middle - 1][2]
    for name, begin, end in last[middle: middle + per_layer]:
        rows.append({"kernel": name, "us": round(end - begin, 1), "adds_us": round(end - previous_end, 1)})
        previous_end = end
    ends = [last[i][2] for i in attention]
    layers = [round(b - a, 1) for a, b in zip(ends, ends[1:])]
    return {"only": "timeline", "batch": batch, "context": start + 8, "kernels_per_step": len(last), "kernels_per_layer": per_layer,
            "layer_us": layers, "step_us": round(last[-1][2] - last[0][1], 1), "one_layer": rows}


def run_4b(args, cfg, model, gen, pk, pk_source) -> dict:
    clocks = ClockSampler()
    check_graph_replay(model, gen)
    main = decode_point(model, args.batch, args.steps, args.warmup, gen, clocks)
    few = max(16, min(64, args.steps // 4))
    # centred on 2,048 and 3,072; at 4,096 the context is full, so those are the last steps that end there
    contexts = {str(label): round(decode_point(model, args.batch, few, args.warmup, gen, centre=centre)["ms_per_step"], 4)
                for label, centre in ((PROMPT, PROMPT), ((PROMPT + CONTEXT) // 2, (PROMPT + CONTEXT) // 2),
                                      (CONTEXT, CONTEXT - few // 2 - 1))}
    prefill = prefill_point(model, gen)
    prefill_eager = prefill_point(model, gen, graphs=False)
    points = {}
    for batch in (1, 64):
        points[f"decode_b{batch}"] = round(decode_point(model, batch, max(16, args.steps // 2), args.warmup, gen)["tok_s"], 1)
    e2e = e2e_point(model, args.batch, max(16, args.steps // 2), args.warmup, gen)
    kernels = kernel_points(args.model, pk, with_library=False) if args.dtype == "bf16" and not args.layers else {}
    achieved = main["bytes"] / (main["ms_per_step"] * 1e-3) / 1e9
    flops = prefill_flops(cfg, cfg.num_hidden_layers, PREFILL_TOKENS)
    tflops_peak = pk["bf16_tflops"] if args.dtype == "bf16" else FP32_TFLOPS
    return {
        "metric": METRIC, "value": round(main["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic token ids, seeded random weights", "impl": "ours",
        "config": config_record(lb_preset(args.model), args.model, cfg.num_hidden_layers, args.batch, PROMPT, CONTEXT,
                                (PROMPT + CONTEXT) // 2, True, pk_source),
        "measured_mean_context": round(main["mean_ctx"]),
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(prefill["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(prefill["ms"], 3),
                    "frac": round(flops / (prefill["ms"] * 1e-3) / (tflops_peak * 1e12), 4),
                    "launch_by_launch_ms": round(prefill_eager["ms"], 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "contexts": contexts,
        "kernels": kernels,
        "graph_check": "replayed step == the same step launch by launch, bit for bit",
        "clocks": clocks.summary(),
    }


def run_4b_fp32(args, cfg, model, gen, pk, pk_source) -> dict:
    """The true 32-bit path at the headline's shape: reported, not the headline."""
    clocks = ClockSampler()
    steps = min(args.steps, 32)
    main = decode_point(model, 8, steps, args.warmup, gen, clocks)
    one = decode_point(model, 1, steps, args.warmup, gen)
    prefill = prefill_point(model, gen, repeats=3)
    flops = prefill_flops(cfg, cfg.num_hidden_layers, PREFILL_TOKENS)
    achieved = main["bytes"] / (main["ms_per_step"] * 1e-3) / 1e9
    return {
        "metric": "decode tokens/s (Qwen3-4B shape, true 32-bit path, batch 8, context 2048->4096)",
        "value": round(main["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic token ids, seeded random weights", "impl": "ours",
        "config": config_record(lb_preset(args.model), args.model, cfg.num_hidden_layers, 8, PROMPT, CONTEXT, main["mean_ctx"],
                                True, pk_source),
        "gpu_launches": main["launches"],
        "points": {"decode_b1": round(one["tok_s"], 1), "decode_b8": round(main["tok_s"], 1)},
        "prefill": {"value": round(prefill["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(prefill["ms"], 3),
                    "frac": round(flops / (prefill["ms"] * 1e-3) / (FP32_TFLOPS * 1e12), 4), "peak_tflops": FP32_TFLOPS},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clocks.summary(),
    }


def run_8b_mixed(args, cfg, model, gen, pk, pk_source) -> dict:
    """32 requests with prompts of 128..8,192 tokens, prompt portions of 2,048 tokens beside decoding
    requests, 512 new tokens each, through `Engine` with captured decode steps and pipelined stepping."""
    import torch
    import layover_b200 as lb

    requests, new_tokens, chunk = 32, 512, 2048
    lengths = torch.randint(128, 8193, (requests,), generator=gen).tolist()
    pages = sum(-(-(n + new_tokens) // PAGE) for n in lengths)
    cache = lb.PagedKVCache(model, pages, block_tokens=PAGE, max_requests=requests)
    engine = lb.Engine(model, cache, lb.EngineConfig(requests, chunk, chunk), cuda_graphs=True)
    # graphs are captured before the clock starts
    engine.step_fn.capture_all(tokens=max(lengths) + new_tokens, from_tokens=min(lengths), skews=(1, 2))
    for i, n in enumerate(lengths):
        engine.add_request(lb.Request(str(i), torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist(), new_tokens))
    clocks = ClockSampler()
    step_ms = []
    torch.cuda.synchronize()
    with clocks:
        began = time.perf_counter()
        last = began
        while not (engine.idle and engine._inflight is None):
            engine.step_pipelined()
            now = time.perf_counter()
            step_ms.append((now - last) * 1e3)
            last = now
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - began
    finished = engine.finished
    if len(finished) != requests or any(len(r.generated) != new_tokens for r in finished):
        raise RuntimeError("bench.py: not every request of the mixed run finished with all its tokens")
    generated = sum(len(r.generated) for r in finished)
    ttft = sorted((r.first_token_at - r.submitted_at) * 1e3 for r in finished)
    step_ms.sort()
    pick = lambda values, q: round(values[min(len(values) - 1, int(q * len(values)))], 2)
    return {
        "metric": "generated tokens/s (Qwen3-8B shape, 32 requests, prompts 128..8192, portions of 2048, 512 new tokens each)",
        "value": round(generated / elapsed, 1), "unit": "tokens/s", "n_gpus": 1, "steps": engine.stats["steps"], "warmup": 0,
        "ms_per_step": round(1e3 * elapsed / max(1, engine.stats["steps"]), 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": args.dtype, "data": "synthetic token ids, seeded random weights", "impl": "ours",
        "config": config_record(lb_preset(args.model), args.model, cfg.num_hidden_layers, requests, sum(lengths) // requests,
                                max(lengths) + new_tokens, sum(lengths) / requests + new_tokens / 2, True, pk_source),
        "seconds": round(elapsed, 3), "prompt_tokens": sum(lengths), "generated_tokens": generated,
        "total_tokens_per_s": round((sum(lengths) + generated) / elapsed, 1),
        "ttft_ms": {"p50": pick(ttft, 0.5), "p90": pick(ttft, 0.9), "max": round(ttft[-1], 2)},
        "step_ms": {"p50": pick(step_ms, 0.5), "p90": pick(step_ms, 0.9), "p99": pick(step_ms, 0.99), "max": round(step_ms[-1], 2)},
        "pool": {"pages": pages, "gib": round(cache.pool_bytes() / 2**30, 2)},
        "engine": dict(engine.stats), "graph_replays": engine.step_fn.graph_replays,
        "gpu_launches": engine.step_fn.replayed_launches,
        "clocks": clocks.summary(),
    }


def run_32b_long(args, cfg, model, gen, pk, pk_source) -> dict:
    """8 prompts of 32,768 tokens, then 256 greedy decode steps timed on the device."""
    batch, prompt, steps = 8, 32768, args.steps
    clocks = ClockSampler()
    began = time.perf_counter()
    point = decode_point(model, batch, steps, args.warmup, gen, clocks, first_ctx=prompt + 1, graph_tokens=prompt + steps + 64)
    achieved = point["bytes"] / (point["ms_per_step"] * 1e-3) / 1e9
    return {
        "metric": "decode tokens/s (Qwen3-32B shape, 8 requests of 32,768-token prompts, 256 greedy steps)",
        "value": round(point["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": round(point["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic token ids, seeded random weights", "impl": "ours",
        "config": config_record(lb_preset(args.model), args.model, cfg.num_hidden_layers, batch, prompt, prompt + steps,
                                point["mean_ctx"], True, pk_source),
        "gpu_launches": point["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(point["bytes"])},
        "seconds_with_prefill": round(time.perf_counter() - began, 1),
        "clocks": clocks.summary(),
    }


def lb_preset(name: str):
    import layover_b200 as lb
    return lb.preset(name)


def parser_default(name: str):
    return {"steps": 256, "warmup": 8}[name]


def run_ours(args) -> dict:
    import torch
    import layover_b200 as lb

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    pk, pk_source = peaks()
    if args.only == "kernels":
        return {"only": "kernels", **kernel_points(args.model, pk, with_library=True)}
    if args.only == "plans":
        return {"only": "plans", **plan_points(args.model, pk)}
    cfg = lb.preset(args.model)
    if args.layers:
        cfg = cfg.replace(num_hidden_layers=args.layers)
    gen = torch.Generator().manual_seed(0)
    model = lb.random_model(cfg, seed=0, device="cuda", dtype=args.dtype, std=0.02)
    if args.only == "decode":
        point = decode_point(model, args.batch, args.steps, args.warmup, gen)
        return {"only": "decode", "batch": args.batch, "layers_run": cfg.num_hidden_layers,
                "tok_s": round(point["tok_s"], 1), "ms_per_step": round(point["ms_per_step"], 4)}
    if args.only == "timeline":
        return {"layers_run": cfg.num_hidden_layers, **timeline_point(model, args.batch, gen)}
    if args.only == "prefill":
        point = prefill_point(model, gen, repeats=max(1, args.steps))
        eager = prefill_point(model, gen, repeats=max(1, args.steps), graphs=False)
        return {"only": "prefill", "layers_run": cfg.num_hidden_layers, "tok_s": round(point["tok_s"], 1),
                "ms": round(point["ms"], 3), "launch_by_launch_ms": round(eager["ms"], 3)}
    runner = {"4b": run_4b, "4b-fp32": run_4b_fp32, "8b-mixed": run_8b_mixed, "32b-long": run_32b_long}[args.config]
    return runner(args, cfg, model, gen, pk, pk_source)


# --------------------------------------------------------------------------------------- the reference
def run_reference(args) -> dict:
    if args.config != "4b":
        return {"impl": "reference", "unavailable": f"the reference arm runs the headline (--config 4b), not {args.config}"}
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
    graphs, graph_width = False, 0
    if backend == "triton" and batch <= 8:
        try:
            from layover.decode_graphs import DecodeGraphs
            model.decode_graphs = DecodeGraphs(model, cache, max_tokens=CONTEXT)
            graphs, graph_width = True, model.decode_graphs.width
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
        first_ctx = max(r.table.num_tokens for r in engine.running)
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
    # what its decode step copies to the device: the packed rows [rows, 3 + table width] of int32
    # (layover/kv/paged_cache.py:154-169, layover/decode_graphs.py:87-91) and the tokens as int64
    if graphs:
        rows = next(s for s in model.decode_graphs.sizes if s >= batch)
        h2d = 4 * rows * (3 + graph_width) + 8 * batch
    else:
        h2d = 4 * batch * (3 + cache.blocks_for(first_ctx + steps)) + 8 * batch
    _, pk_source = peaks()
    return {
        "metric": METRIC, "value": round(batch * 1000.0 / device_ms, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(device_ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, torch default random weights", "impl": "reference",
        # (the contexts its timed steps really had are a few tokens longer: requests that finish their prompt early
        # decode while the others still prefill; `measured_mean_context` says by how much)
        "config": config_record(ours, args.model, cfg.num_hidden_layers, batch, PROMPT, CONTEXT,
                                (PROMPT + CONTEXT) // 2, graphs, pk_source),
        "measured_mean_context": round(first_ctx + (steps + 1) / 2),
        "decode_backend": backend,
        "e2e": {"value": round(produced / elapsed, 2), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 8 * batch},
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3)},
        "clocks": clocks.summary(),
    }


def main(argv=None) -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=parser_default("steps"))
    parser.add_argument("--warmup", type=int, default=parser_default("warmup"))
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--config", default="4b", choices=sorted(CONFIGS),
                        help="4b: the headline; 4b-fp32: the 32-bit path; 8b-mixed: 32 mixed requests through the "
                             "scheduler; 32b-long: 8 x 32,768-token contexts")
    parser.add_argument("--model", default=None, help="a preset's name instead of the one --config names")
    parser.add_argument("--dtype", default=None, choices=["bf16", "fp32"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="run fewer layers than the shape has (both numbers are reported)")
    parser.add_argument("--only", default="all", choices=["all", "decode", "prefill", "kernels", "timeline", "plans"],
                        help="decode or prefill alone, as a small target for a profiler; the dominant kernels alone "
                             "with cuBLAS beside them; one replayed decode step's time kernel by kernel; or the "
                             "decode attention over its launch plans for equal and unequal lengths (each prints a "
                             "short line)")
    args = parser.parse_args(argv)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    model, dtype = CONFIGS[args.config]
    args.model = args.model or model
    args.dtype = args.dtype or dtype
    args.warmup = max(3, args.warmup)
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
