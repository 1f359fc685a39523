"""The path that serving and the benchmark time, compared with the plain implementation: decode
steps replayed from captured CUDA graphs (padded to a bucket of requests), the head size of the
served models, dozens to more than a hundred requests decoding together, the 4B layer shape in
both precisions, pipelined stepping, and a checkpoint stored in 32-bit run in bfloat16."""

import json

import numpy as np
import pytest
import torch

import layover_b200 as lb
from conftest import TINY, TINY_PAGE, random_prompt, tolerance
from plain_qwen3 import plain_forward
from replay_helpers import crowd, mixed, portions, run_trace, tail_decoded, whole
from test_gpu_replay import CUTS, DTYPES, compare, expected_rows, requests_for

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------ graphs on, every cut
@pytest.mark.parametrize("name,dtype_name", [("c", "bfloat16"), ("d", "bfloat16"), ("a", "float32"), ("b", "float32")])
@pytest.mark.parametrize("cut", ["tail", "mixed", "crowd"])
def test_cuts_with_captured_decode_steps(tiny_folders, tmp_path, name, dtype_name, cut):
    """Steps of single tokens replay a captured graph: one request alone (bucket 1), three of four
    live requests (bucket 4, one padded row), five to six of eight (bucket 8)."""
    folder, _, _ = tiny_folders[name]
    requests = requests_for(name)
    if cut == "crowd":
        steps = crowd(requests, decoded=7, prompts_per_step=3)
        sizes = {len(s["entries"]) for s in steps if all(len(e["tokens"]) == 1 for e in s["entries"])}
        assert 5 in sizes or 6 in sizes                   # rows that are no bucket size: padded rows run
    else:
        steps = CUTS[cut](requests)
    if cut == "mixed":
        sizes = {len(s["entries"]) for s in steps if all(len(e["tokens"]) == 1 for e in s["entries"])}
        assert 3 in sizes
    rows = run_trace(folder, dtype_name, steps, tmp_path, block_tokens=TINY_PAGE[name], cuda_graphs=True)
    compare(rows, expected_rows(tiny_folders, name, dtype_name), DTYPES[dtype_name])


def test_a_replayed_step_equals_the_same_launches_without_a_graph(tiny_folders):
    """Replay against the graph's own fixed-size batch run launch by launch: bit for bit, with the
    sampled tokens and the requests' records, at the served head size in bfloat16 with padded rows."""
    from layover_b200.engine.step import StepFunction

    folder, _, _ = tiny_folders["c"]
    model = lb.load_model(folder, device="cuda", dtype="bf16")
    outputs = []
    for replay in (True, False):
        cache = lb.PagedKVCache(model, 64, block_tokens=16, max_requests=8)
        step = StepFunction(model, cache, cuda_graphs=True)
        step.replay_graphs = replay
        seqs = [cache.open(f"r{i}") for i in range(3)]
        for i, seq in enumerate(seqs):
            step([lb.StepEntry(seq, random_prompt(384, 20 + 37 * i, 60 + i), [])])
        got = []
        for turn in range(5):
            logits = step([lb.StepEntry(seq, [(7 * turn + i) % 384], [0]) for i, seq in enumerate(seqs)]).clone()
            tokens = step.sample([lb.StepEntry(seq, [lb.DEVICE_TOKEN], [0]) for seq in seqs]).result()
            got.append((logits.cpu(), tokens))
        assert step.graph_replays == (10 if replay else 0)
        outputs.append((got, cache.records.cpu().clone()))
    (with_graph, records_a), (without, records_b) = outputs
    for (la, ta), (lb_, tb) in zip(with_graph, without):
        assert torch.equal(la, lb_) and ta == tb
    assert torch.equal(records_a, records_b)


@pytest.mark.parametrize("name,dtype_name", [("c", "bf16"), ("b", "fp32")])
def test_a_captured_prompt_portion_equals_the_same_launches_without_a_graph(tiny_folders, name, dtype_name):
    """A prompt cut into portions of the captured size (and a shorter rest): the portions replay a
    graph, one that wants no logits and one that wants the last token's; logits, sampled token, cache
    contents and record equal the same steps run launch by launch, and the plain implementation."""
    from layover_b200.engine.step import StepFunction

    folder, raw, weights = tiny_folders[name]
    model = lb.load_model(folder, device="cuda", dtype=dtype_name)
    page, size = TINY_PAGE[name], 48
    vocab = raw["vocab_size"]
    prompt = random_prompt(vocab, 3 * size + 11, 77)
    outputs = []
    for graphs in (True, False):
        cache = lb.PagedKVCache(model, 4 * (len(prompt) // page + 2), block_tokens=page, max_requests=2)
        step = StepFunction(model, cache, cuda_graphs=graphs, portion_graph_tokens=(size,))
        got = []
        for round_ in range(2):                       # the second request runs on pages and a graph used before
            seq = cache.open(f"r{round_}")
            step([lb.StepEntry(seq, prompt[:size], [])])
            got.append(step([lb.StepEntry(seq, prompt[size:2 * size], [size - 1])]).clone().cpu())
            tokens = step.sample([lb.StepEntry(seq, prompt[2 * size:3 * size], [size - 1])]).result()
            got.append(step([lb.StepEntry(seq, prompt[3 * size:], [10])]).clone().cpu())
            got.append(torch.tensor(tokens))
            if round_ == 0:
                cache.close(seq)
        assert step.graph_replays == (6 if graphs else 0)
        outputs.append((got, cache.records[: cache.max_requests].cpu().clone()))    # not the scratch record
    (with_graph, records_a), (without, records_b) = outputs
    for a, b in zip(with_graph, without):
        assert torch.equal(a, b)
    assert torch.equal(records_a, records_b)
    dtype = torch.bfloat16 if dtype_name == "bf16" else torch.float32
    plain = plain_forward(raw, weights, prompt, dtype)
    for got_row, place in ((with_graph[0][0], 2 * size - 1), (with_graph[1][0], len(prompt) - 1)):
        assert (got_row - plain[place]).abs().max() <= tolerance(plain[place], dtype)
    token, row = int(with_graph[2][0]), plain[3 * size - 1]
    assert row[token] >= row.max() - tolerance(row, dtype)


# ------------------------------------------------------------------ many requests decoding together
@pytest.mark.parametrize("dtype_name", ["bfloat16", "float32"])
@pytest.mark.parametrize("count", [24, 64, 130])
def test_many_requests_decoding_together(tiny_folders, tmp_path, dtype_name, count):
    """Decode steps of 24, 64 and 130 rows (the matrix products' 17..128-token and > 128-token paths,
    the separate per-head norm and activation kernels) against the plain implementation."""
    folder, raw, weights = tiny_folders["c"]
    requests = {f"m{i}": random_prompt(384, 9 + (5 * i) % 23, 7000 + i) for i in range(count)}
    steps = crowd(requests, decoded=4, prompts_per_step=32)
    assert max(len(s["entries"]) for s in steps) == count
    rows = run_trace(folder, dtype_name, steps, tmp_path, block_tokens=16, max_requests=count,
                     cuda_graphs=(count <= 64))
    expected = {rid: plain_forward(raw, weights, tokens, DTYPES[dtype_name]).numpy() for rid, tokens in requests.items()}
    compare(rows, expected, DTYPES[dtype_name])


# ------------------------------------------------------------------ the engine with graphs and pipelined stepping
def test_engine_with_graphs_and_pipelining_at_the_served_head_size(tiny_folders):
    """Tiny C in bfloat16 through `Engine`: captured decode steps and pipelined stepping give, token
    for token, what the same fixed-size steps give launch by launch with every token read at once;
    and every token is the best under the plain implementation's logits for its own prefix, give or
    take the bfloat16 tolerance."""
    folder, raw, weights = tiny_folders["c"]
    model = lb.load_model(folder, device="cuda", dtype="bf16")
    prompts = [random_prompt(384, n, 400 + n) for n in (5, 140, 33, 61, 18)]
    results = []
    for pipelined in (True, False):
        cache = lb.PagedKVCache(model, 96, block_tokens=16, max_requests=4)
        engine = lb.Engine(model, cache, lb.EngineConfig(max_batch=3, prefill_chunk=64, prefill_budget=64), cuda_graphs=True)
        engine.step_fn.replay_graphs = pipelined
        for i, p in enumerate(prompts):
            engine.add_request(lb.Request(str(i), p, 14, temperature=0.7 if i == 1 else 0.0, seed=3))
        if pipelined:
            engine.run_until_idle()
            assert engine.step_fn.graph_replays > 10
        else:
            while not engine.idle:
                engine.step()
        assert cache.num_free == 96
        cache.check()
        results.append({r.request_id: r.generated for r in engine.finished})
    assert results[0] == results[1]
    for i, prompt in enumerate(prompts):
        if i == 1:
            continue                                   # drawn at a temperature; pinned by the fp32 sampling tests
        seq = list(prompt)
        for token in results[0][str(i)]:
            logits = plain_forward(raw, weights, seq, torch.bfloat16)[-1]
            assert logits[token] >= logits.max() - tolerance(logits, torch.bfloat16)
            seq.append(token)


# ------------------------------------------------------------------ the 4B layer shape, both precisions, every cut
@pytest.fixture(scope="module")
def layer_4b(tmp_path_factory):
    from safetensors.torch import load_file

    config = lb.Qwen3Config(vocab_size=512, hidden_size=2560, intermediate_size=9728, num_hidden_layers=2,
                            num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=1024,
                            rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
    folder = tmp_path_factory.mktemp("layer-4b")
    lb.write_model_folder(config, folder, seed=21, std=0.02, norm_std=0.1)
    raw = json.loads((folder / "config.json").read_text())
    weights = load_file(str(folder / "model.safetensors"))
    requests = {f"r{i}": random_prompt(512, n, 950 + i) for i, n in enumerate([150, 9, 70, 40, 133])}
    return folder, raw, weights, requests


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_every_cut_at_the_4b_layer_shape(layer_4b, tmp_path, dtype_name):
    folder, raw, weights, requests = layer_4b
    dtype = DTYPES[dtype_name]
    expected = {rid: plain_forward(raw, weights, tokens, dtype).numpy() for rid, tokens in requests.items()}
    base = None
    for cut in ("whole", "tail", "portions", "mixed"):
        steps = CUTS[cut](requests)
        rows = run_trace(folder, dtype_name, steps, tmp_path / cut, block_tokens=16, cuda_graphs=(cut == "tail"))
        compare(rows, expected, dtype)
        if dtype_name == "float32":                    # every sum has a fixed order: cutting changes no bit
            if base is None:
                base = rows
            else:
                for rid in requests:
                    for position, row in base[rid].items():
                        assert np.array_equal(rows[rid][position], row), f"{cut}: {rid} position {position} differs"


def test_long_portions_at_the_4b_layer_shape(layer_4b, tmp_path):
    """Portions of 512 tokens and more take the products on pairs of blocks and the q/k/v projection
    with the norm, the rotation and the page write in its epilogue; shorter ones the single-block
    products and the per-head kernel. A 900-token prompt whole, as 600 + 300 and as three times 300,
    and 600 of it beside two other requests' single tokens: the wanted rows against the plain
    implementation, and the three cuts against one another."""
    folder, raw, weights, _ = layer_4b
    long = random_prompt(512, 900, 4242)
    short = {"s0": random_prompt(512, 20, 1), "s1": random_prompt(512, 35, 2)}
    wanted = [0, 1, 299, 300, 511, 512, 599, 600, 898, 899]

    def cut(sizes):
        steps, at = [], 0
        for size in sizes:
            want = [w - at for w in wanted if at <= w < at + size]
            steps.append({"entries": [{"id": "long", "tokens": long[at:at + size], "want": want}], "end": []})
            at += size
        steps[-1]["end"] = ["long"]
        return [dict(step, step=i) for i, step in enumerate(steps)]

    beside = [{"step": 0, "entries": [{"id": rid, "tokens": tokens[:-1], "want": []} for rid, tokens in short.items()], "end": []},
              {"step": 1, "entries": [{"id": "long", "tokens": long[:600], "want": [w for w in wanted if w < 600]}] +
                                     [{"id": rid, "tokens": tokens[-1:], "want": [0]} for rid, tokens in short.items()],
               "end": ["s0", "s1"]},
              {"step": 2, "entries": [{"id": "long", "tokens": long[600:], "want": [w - 600 for w in wanted if w >= 600]}],
               "end": ["long"]}]
    plain = plain_forward(raw, weights, long, torch.bfloat16)
    expected = {"long": plain.numpy()}
    expected.update({rid: plain_forward(raw, weights, tokens, torch.bfloat16).numpy() for rid, tokens in short.items()})
    results = {}
    for name, steps in (("whole", cut([900])), ("600+300", cut([600, 300])), ("3x300", cut([300, 300, 300])), ("beside", beside)):
        rows = run_trace(folder, "bfloat16", steps, tmp_path / name, block_tokens=16, max_tokens=1100)
        assert sorted(rows["long"]) == wanted
        for rid, got in rows.items():
            bound = tolerance(torch.from_numpy(expected[rid]), torch.bfloat16)
            for position, row in got.items():
                worst = np.abs(row - expected[rid][position]).max()
                assert worst <= bound, f"{name}: {rid} position {position}: |diff| {worst:.3e} > {bound:.3e}"
        if name == "beside":
            assert sorted(rows["s0"]) == [19] and sorted(rows["s1"]) == [34]
        results[name] = rows["long"]
    bound = tolerance(plain, torch.bfloat16)
    for name in ("600+300", "3x300", "beside"):
        for position in wanted:
            assert np.abs(results[name][position] - results["whole"][position]).max() <= bound


# ------------------------------------------------------------------ a checkpoint stored in 32-bit, run in bfloat16
def test_a_32bit_checkpoint_run_in_bfloat16(tmp_path):
    """Every floating tensor is rounded to the run's dtype when it is loaded, the norm weights too
    (layover/weights.py:35): values that bfloat16 cannot hold must give the plain implementation's
    bfloat16 logits, not those of unrounded norm weights."""
    from safetensors.torch import load_file

    config = lb.Qwen3Config(**TINY["b"])
    lb.write_model_folder(config, tmp_path, seed=77, std=0.05, norm_std=0.2, store_dtype=torch.float32)
    raw = json.loads((tmp_path / "config.json").read_text())
    weights = load_file(str(tmp_path / "model.safetensors"))
    norm = weights["model.layers.0.input_layernorm.weight"]
    assert norm.dtype == torch.float32 and not torch.equal(norm, norm.to(torch.bfloat16).float())
    requests = {"x": random_prompt(512, 90, 1), "y": random_prompt(512, 33, 2)}
    rows = run_trace(tmp_path, "bfloat16", tail_decoded(requests, 8), tmp_path / "out", block_tokens=16)
    expected = {rid: plain_forward(raw, weights, tokens, torch.bfloat16).numpy() for rid, tokens in requests.items()}
    compare(rows, expected, torch.bfloat16)
    model = lb.load_model(tmp_path, device="cuda", dtype="bf16")
    held = model.blocks[0].input_norm.weight
    assert held.dtype == torch.float32 and torch.equal(held.cpu(), norm.to(torch.bfloat16).float())


# ------------------------------------------------------------------ what the kernels cannot check is checked before them
def test_a_corrupt_table_is_refused_before_any_launch(tiny_folders):
    """A page id outside the pool, a page the request does not hold, a table too short for its
    tokens, a request of another cache: each is refused on the host, no kernel has run, and the
    cache is as it was (layover/kv/paged_cache.py:160-165 refuses the same before its launches)."""
    from layover_b200 import ops
    from layover_b200.engine.step import StepFunction

    folder, _, _ = tiny_folders["a"]
    model = lb.load_model(folder, device="cuda", dtype="fp32")
    cache = lb.PagedKVCache(model, 16, block_tokens=4, max_requests=4)
    step = StepFunction(model, cache)
    seq = cache.open("v")
    step([lb.StepEntry(seq, random_prompt(256, 10, 1), [])])
    good = list(seq.tables[0].blocks)
    free_page = next(p for p in range(16) if not cache.paged[0].allocator.is_held(p))
    for bad, message in ((9999, "outside its pool"), (-3, "outside its pool"), (free_page, "not an allocated page")):
        seq.tables[0].blocks[1] = bad
        launches = ops.LAUNCHES
        with pytest.raises(ValueError, match=message):
            step([lb.StepEntry(seq, [5], [0])])
        assert ops.LAUNCHES == launches and seq.num_tokens == 10
        seq.tables[0].blocks[:] = good
    with pytest.raises(ValueError, match="not an allocated page"):
        seq.tables[0].blocks[0] = free_page
        cache.check_tables(seq)
    seq.tables[0].blocks[:] = good
    cache.check_tables(seq)
    other = lb.PagedKVCache(model, 16, block_tokens=4, max_requests=4)
    stranger = other.open("v2")
    with pytest.raises(ValueError, match="does not belong"):
        step([lb.StepEntry(stranger, [5], [0])])
    logits = step([lb.StepEntry(seq, [5], [0])])          # and the cache still works
    assert logits.shape == (1, 256) and torch.isfinite(logits).all()
    cache.check()


# ------------------------------------------------------------------ a kernel that gave up is heard of, and the engine recovers
def test_a_wait_that_ran_out_reaches_the_host_with_the_tokens_and_the_engine_recovers(tiny_folders):
    """Every wait in the tensor-core kernels is bounded; a wait that runs out leaves a code in the
    library's error word and may leave split counters that are not back at zero. Nothing is made to
    hang here: the test writes the code and dirty counters from the host, as such a kernel would leave
    them. The sampling kernel carries the word to the host behind the step's tokens: the step's tokens
    are refused with a KernelError, words and counters are put back, and generation goes on correctly."""
    from layover_b200 import ops

    folder, raw, weights = tiny_folders["c"]
    model = lb.load_model(folder, device="cuda", dtype="bf16")
    prompts = [random_prompt(384, n, 500 + n) for n in (12, 40)]
    clean = lb.generate(model, prompts, max_new_tokens=6, block_tokens=16)
    cache = lb.PagedKVCache(model, 32, block_tokens=16, max_requests=4)
    engine = lb.Engine(model, cache, lb.EngineConfig(max_batch=2, prefill_chunk=64, prefill_budget=64))
    for i, p in enumerate(prompts):
        engine.add_request(lb.Request(str(i), p, 6))
    engine.step()                                              # both prompts, first tokens
    ops.gemm_set_status(4)                                     # "the split sum's wait ran out"
    partials, counters, _ = ops.gemm_scratch(model.device)
    counters[:8] = 3                                           # counters a block that gave up did not put back
    with pytest.raises(ops.KernelError, match="gemm_tcgen05: code 4"):
        engine.step()
    assert ops.gemm_status() == 0 and int(counters.abs().sum()) == 0      # cleared before the error was raised
    # a fresh engine on the same device runs the same requests to the same tokens
    again = lb.generate(model, prompts, max_new_tokens=6, block_tokens=16)
    assert again == clean
