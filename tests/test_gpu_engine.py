"""The engine on the GPU above the step function: greedy and temperature generation through the
Python entry point and the command line, long decoding, the first tokens of a sequence, captured
decode steps, each part alone, and parts that are not Qwen3's (a window, a layer that reads
another layer's pages, a layer that runs twice, a toy mixer with state of its own)."""

import json
import math
import subprocess
import sys

import numpy as np
import pytest
import torch

import layover_b200 as lb
from conftest import ROOT, TINY, TINY_PAGE, random_prompt, tolerance
from plain_qwen3 import plain_forward, plain_generate, plain_mlp, plain_rmsnorm, plain_sample

pytestmark = pytest.mark.gpu

DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16}


@pytest.fixture(scope="module")
def models(tiny_folders):
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = lb.load_model(tiny_folders[name][0], device="cuda", dtype=dtype)
        return cache[(name, dtype)]
    return get


def test_greedy_generation_matches_the_plain_implementation(tiny_folders, models):
    for name, lengths, steps in (("a", [5, 17, 33], 16), ("b", [1, 9, 64, 130], 24)):
        _, raw, weights = tiny_folders[name]
        prompts = [random_prompt(TINY[name]["vocab_size"], n, 40 + n) for n in lengths]
        expected = [plain_generate(raw, weights, p, steps) for p in prompts]
        config = lb.EngineConfig(max_batch=4, prefill_chunk=32, prefill_budget=32)
        got = lb.generate(models(name, "fp32"), prompts, max_new_tokens=steps, block_tokens=TINY_PAGE[name], config=config)
        assert got == expected
        graphs = lb.generate(models(name, "fp32"), prompts, max_new_tokens=steps, block_tokens=TINY_PAGE[name],
                             config=config, cuda_graphs=True)
        assert graphs == expected


def test_bf16_generation_stays_on_the_plain_models_best_tokens(tiny_folders, models):
    _, raw, weights = tiny_folders["b"]
    prompts = [random_prompt(512, n, 7 + n) for n in (9, 64)]
    got = lb.generate(models("b", "bf16"), prompts, max_new_tokens=12, block_tokens=16)
    for prompt, tokens in zip(prompts, got):
        seq = list(prompt)
        for token in tokens:
            logits = plain_forward(raw, weights, seq, torch.bfloat16)[-1]
            assert logits[token] >= logits.max() - tolerance(logits, torch.bfloat16)
            seq.append(token)


def test_temperature_sampling_is_the_plain_rule_and_ignores_the_batch(tiny_folders, models):
    _, raw, weights = tiny_folders["b"]
    model = models("b", "fp32")
    prompts = [random_prompt(512, n, 90 + n) for n in (1, 9, 64, 130)]
    config = lb.EngineConfig(max_batch=4, prefill_chunk=32, prefill_budget=32)
    together = lb.generate(model, prompts, max_new_tokens=24, temperature=0.8, seed=5, block_tokens=16, config=config)
    for index, prompt in enumerate(prompts):
        alone = lb.generate(model, [prompt], max_new_tokens=24, temperature=0.8, seed=5 + index, block_tokens=16)
        assert alone[0] == together[index]
        seq = list(prompt)
        for step, token in enumerate(together[index]):       # each draw follows the plain rule on the plain logits
            logits = plain_forward(raw, weights, seq).numpy()[-1]
            assert token == plain_sample(logits, 0.8, 5 + index, step)
            seq.append(token)
    assert together != lb.generate(model, prompts, max_new_tokens=24, temperature=0.8, seed=6, block_tokens=16, config=config)


def test_pipelined_stepping_equals_step_by_step_and_handles_stop_tokens(tiny_folders, models):
    """`run_until_idle` launches each step before it has read the tokens of the one before; `step`
    waits for its own tokens. Both must give the plain implementation's tokens, also when a request
    ends on a stop token (found out one step late, with one token in flight that is dropped)."""
    _, raw, weights = tiny_folders["b"]
    model = models("b", "fp32")
    prompts = [random_prompt(512, n, 300 + n) for n in (3, 20, 70, 9)]
    expected = [plain_generate(raw, weights, p, 12) for p in prompts]
    stops = [frozenset({expected[0][4]}), frozenset(), frozenset({expected[2][0]}), frozenset({expected[3][11]})]
    cut = []
    for tokens, stop in zip(expected, stops):
        end = next((i for i, t in enumerate(tokens) if t in stop), len(tokens) - 1)
        cut.append(tokens[:end + 1])
    for pipelined in (True, False):
        for graphs in (False, True):
            cache = lb.PagedKVCache(model, 64, block_tokens=16, max_requests=4)
            engine = lb.Engine(model, cache, lb.EngineConfig(max_batch=3, prefill_chunk=16, prefill_budget=24), cuda_graphs=graphs)
            for i, (p, stop) in enumerate(zip(prompts, stops)):
                engine.add_request(lb.Request(str(i), p, 12, stop))
            if pipelined:
                engine.run_until_idle()
            else:
                while not engine.idle:
                    engine.step()
            done = {r.request_id: r.generated for r in engine.finished}
            assert [done[str(i)] for i in range(4)] == cut
            assert cache.num_free == 64 and all(r.pending == 0 for r in engine.finished)
            cache.check()
            if pipelined:
                assert engine.stats["dropped_tokens"] >= 1      # the steps in flight behind the stop tokens


def test_long_decoding_and_page_reuse(tiny_folders, models):
    _, raw, weights = tiny_folders["a"]
    model = models("a", "fp32")
    cache = lb.PagedKVCache(model, 64, block_tokens=4, max_requests=4)
    engine = lb.Engine(model, cache, lb.EngineConfig(max_batch=2, prefill_chunk=8, prefill_budget=8))
    prompts = [random_prompt(256, n, n) for n in (6, 11, 3, 20)]
    for i, p in enumerate(prompts):
        engine.add_request(lb.Request(str(i), p, 200))      # 200 tokens token by token; two waves share the pages
    done = {r.request_id: r.generated for r in engine.run_until_idle()}
    for i, p in enumerate(prompts):
        assert done[str(i)] == plain_generate(raw, weights, p, 200)
    assert cache.num_free == 64
    cache.check()


def test_first_tokens_of_a_sequence(tiny_folders, tmp_path):
    from replay_helpers import run_trace
    for name in ("a", "b"):
        folder, raw, weights = tiny_folders[name]
        for dtype_name, dtype in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            tokens = random_prompt(TINY[name]["vocab_size"], 6, 1)
            steps = [{"step": i, "entries": [{"id": "f", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(tokens)]
            rows = run_trace(folder, dtype_name, steps, tmp_path / f"{name}{dtype_name}", block_tokens=TINY_PAGE[name])
            reference = plain_forward(raw, weights, tokens, dtype).numpy()
            got = np.stack([rows["f"][i] for i in range(6)])
            assert np.abs(got - reference).max() <= tolerance(torch.from_numpy(reference), dtype)


def test_command_line(tiny_folders):
    folder, raw, weights = tiny_folders["a"]
    out = subprocess.run([sys.executable, "-m", "layover_b200", "--model", str(folder), "--dtype", "fp32",
                          "--prompt-ids", "5,17,3", "--prompt-ids", "9", "--max-new-tokens", "5", "--num-blocks", "32",
                          "--block-tokens", "4", "--max-batch", "2", "--prefill-chunk", "2"],
                         capture_output=True, text=True, cwd=ROOT, check=True)
    result = json.loads(out.stdout.strip().splitlines()[-1])
    assert result["generated"] == [plain_generate(raw, weights, p, 5) for p in ([5, 17, 3], [9])]
    assert result["stats"]["prefill_tokens"] == 4


# ------------------------------------------------------------------ each part alone
def runtime(dtype):
    from layover_b200.models.runtime import make_runtime
    return make_runtime(dtype, "cuda")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part_alone(dtype):
    from layover_b200.parts import PartSpec, build_part
    norm = build_part("norm", PartSpec("rmsnorm", {"dim": 200, "eps": 1e-4, "weight": "w"}), "p.")
    assert [(s.name, s.shape, s.kind) for s in norm.tensor_specs()] == [("p.w", (200,), "vector")]
    weight = (1 + 0.3 * torch.randn(200)).to(dtype)
    norm.bind({"p.w": weight.float().cuda()}, runtime(dtype))
    x, delta = torch.randn(9, 200).to(dtype), torch.randn(9, 200).to(dtype)
    stream = x.clone().cuda()
    got = norm.forward(stream, delta.cuda())
    expected = plain_rmsnorm((x.float() + delta.float()).to(dtype), weight, 1e-4)
    assert (got.float().cpu() - expected.float()).abs().max() <= tolerance(expected.float(), dtype)
    assert torch.equal(stream.cpu(), (x.float() + delta.float()).to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part_alone(dtype):
    from layover_b200.parts import PartSpec, build_part
    ffn = build_part("feed_forward", PartSpec("gated_mlp", {"hidden": 72, "inter": 150, "gate": "g", "up": "u", "down": "d"}), "m.")
    assert sorted((s.name, s.shape) for s in ffn.tensor_specs()) == [("m.d", (72, 150)), ("m.g", (150, 72)), ("m.u", (150, 72))]
    w = {k: (torch.randn(*s) / math.sqrt(s[1])).to(dtype) for k, s in (("m.g", (150, 72)), ("m.u", (150, 72)), ("m.d", (72, 150)))}
    ffn.bind({k: v.cuda() for k, v in w.items()}, runtime(dtype))
    h = torch.randn(13, 72).to(dtype)
    got = ffn.forward(h.cuda())
    expected = plain_mlp(h, w["m.g"], w["m.u"], w["m.d"])
    assert (got.float().cpu() - expected.float()).abs().max() <= tolerance(expected.float(), dtype)


def test_position_part_alone():
    from layover_b200.parts import PartSpec, build_part
    rope = build_part("position", PartSpec("rotary_half", {"dim": 48, "theta": 12345.0}), "")
    rope.bind({}, runtime(torch.float32))
    expected = 1.0 / (12345.0 ** (torch.arange(0, 48, 2, dtype=torch.float32) / 48))
    assert torch.equal(rope.inv_freq().cpu(), expected)
    from types import SimpleNamespace
    batch = SimpleNamespace(n_tokens=3, positions=torch.tensor([0, 7, 300], dtype=torch.int32, device="cuda"), shared={})
    table = rope.tables(batch)
    angles = torch.tensor([0.0, 7.0, 300.0])[:, None] * expected[None, :]
    assert (table[:, 0].cpu() - angles.cos()).abs().max() < 1e-5 and (table[:, 1].cpu() - angles.sin()).abs().max() < 1e-5
    assert rope.tables(batch) is table               # made once per step, then shared
    with pytest.raises(ValueError, match="unknown position kind"):
        build_part("position", PartSpec("alibi", {}), "")


# ------------------------------------------------------------------ other arrangements of the same parts
def toy_spec(cfg, window=None, schedule=None, shares=()):
    """Qwen3's parts in other arrangements: a window on every layer, another layer order, layers
    without k/v projections that read an earlier layer's pages."""
    from layover_b200.models import ScheduleEntry
    from layover_b200.models.qwen3 import qwen3_spec
    from layover_b200.parts import PartSpec

    spec = qwen3_spec(cfg)
    layers = []
    for index, layer in enumerate(spec.layers):
        params = dict(layer.block.params)
        mixer = dict(params["mixer"].params)
        mixer["window"] = window
        mixer["shares_cache"] = index in shares
        params["mixer"] = PartSpec("attention", mixer)
        layers.append(type(layer)(PartSpec("pre_norm", params), layer.prefix))
    spec.layers = layers
    if schedule:
        spec.schedule = [ScheduleEntry(layer, reads) for layer, reads in schedule]
    return spec


def build_toy(tiny_folders, name, dtype, **changes):
    from layover_b200.models.model import assemble
    from layover_b200.models.runtime import make_runtime
    from layover_b200.weights import load_tensors

    folder, raw, weights = tiny_folders[name]
    cfg = lb.Qwen3Config.from_hf_dict(raw)
    spec = toy_spec(cfg, **changes)
    model = assemble(spec, cfg)
    wanted = model.tensor_specs()
    stored = {s.name for s in wanted}
    tensors = load_tensors(folder, wanted, dtype, "cuda", ignorable=set(weights) - stored)
    return model.bind(tensors, make_runtime(dtype, "cuda")), raw, weights


def step_in_portions(model, tokens, page, cuts, blocks=64):
    from layover_b200.engine.step import StepFunction
    cache = lb.PagedKVCache(model, blocks, block_tokens=page, max_requests=2)
    step, seq, rows, at = StepFunction(model, cache), None, [], 0
    seq = cache.open("t")
    for size in cuts:
        part = tokens[at:at + size]
        if not part:
            break
        rows.append(step([lb.StepEntry(seq, part, list(range(len(part))))]).cpu())
        at += len(part)
    assert at == len(tokens)
    return torch.cat(rows), cache, seq


@pytest.mark.parametrize("window", [3, 16, 21])
def test_window_layers_match_the_plain_window_and_give_pages_back(tiny_folders, window):
    model, raw, weights = build_toy(tiny_folders, "a", torch.float32, window=window)
    tokens = random_prompt(256, 90, window)
    got, cache, seq = step_in_portions(model, tokens, 4, [7, 2, 30, 1, 1, 1, 17, 2, 29], blocks=16)
    expected = plain_forward(raw, weights, tokens, window=window)
    assert (got - expected).abs().max() <= tolerance(expected, torch.float32)
    assert cache.paged[0].allocator.num_used <= (window + 3) // 4 + 1      # 90 tokens would hold 23 pages
    cache.close(seq)
    assert cache.num_free == 16


def test_a_layer_may_run_twice_and_a_layer_may_read_another_layers_pages(tiny_folders):
    schedule = [(0, None), (1, None), (2, 0), (1, None)]      # layer 2 attends over entry 0's pages; layer 1 runs twice
    model, raw, weights = build_toy(tiny_folders, "b", torch.float32, schedule=schedule, shares=(2,))
    names = {s.name for s in model.tensor_specs()}
    assert "model.layers.2.self_attn.k_proj.weight" not in names and "model.layers.2.self_attn.q_proj.weight" in names
    needs = model.cache_needs()
    assert [n[2] for n in needs] == [None, None, 0, None]
    tokens = random_prompt(512, 50, 2)
    got, cache, _ = step_in_portions(model, tokens, 16, [20, 1, 1, 28])
    assert cache.paged[0].pool.shape[0] == 3                   # three entries own pages, the reader none
    expected = plain_forward(raw, weights, tokens, schedule=schedule)
    assert (got - expected).abs().max() <= tolerance(expected, torch.float32)


# ------------------------------------------------------------------ a toy mixer with state of its own
@pytest.mark.parametrize("own_kernel", [False, True])
def test_a_toy_mixer_with_its_own_state_registers_builds_and_steps(tmp_path, own_kernel):
    """A mixer defined here, not in the package: a per-request running mean of the inputs, kept in
    a fixed-size state slot, projected by one matrix. Registered, built from a model folder and
    stepped through the same step function, with no change to the package. With `own_kernel` its
    forward launches a CUDA kernel of its own, from a source file of this test folder that it
    registers with the package's builder and names in `kernel_libraries`: it is compiled with the
    model's other kernels before the first step."""
    import ctypes

    from layover_b200.csrc import build
    from layover_b200.config import register_architecture, unregister_architecture
    from layover_b200.engine.step import StepFunction
    from layover_b200.models import ModelSpec, LayerSpec
    from layover_b200.parts import Part, PartSpec, StateNeed, register_mixer, unregister
    from layover_b200.weights import TensorSpec

    class RunningMean(Part):
        def __init__(self, params, prefix):
            super().__init__(params, prefix)
            self.hidden = params["hidden"]
            self.name = prefix + "mean_proj.weight"

        def tensor_specs(self):
            return [TensorSpec(self.name, (self.hidden, self.hidden))]

        def cache_need(self):
            return StateNeed((self.hidden + 1,), torch.float32)      # the sum so far and the count

        def bind(self, tensors, runtime):
            super().bind(tensors, runtime)
            self.weight = tensors[self.name]

        def kernel_libraries(self, dtype):
            return ("toy_running_mean",) if own_kernel else ()

        def forward(self, h, batch, cache):
            out = torch.empty_like(h)
            if own_kernel:
                fn = build.load("toy_running_mean").toy_running_mean
                fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
                code = fn(h.data_ptr(), out.data_ptr(), cache.state.data_ptr(), batch.cu_q.data_ptr(),
                          batch.state_slots.data_ptr(), batch.n_seqs, self.hidden, torch.cuda.current_stream().cuda_stream)
                assert code == 0
                return self.runtime.linear(out, self.weight)
            cu, slots = batch.cu_q.tolist(), batch.state_slots.tolist()   # a toy may read back; the engine's parts do not
            for s in range(batch.n_seqs):
                rows = h[cu[s]:cu[s + 1]].float()
                state = cache.state[slots[s]]
                sums = state[:-1] + rows.cumsum(0)
                counts = state[-1] + torch.arange(1, rows.shape[0] + 1, device=h.device)
                out[cu[s]:cu[s + 1]] = (sums / counts[:, None]).to(h.dtype)
                state[:-1], state[-1] = sums[-1], counts[-1]
            return self.runtime.linear(out, self.weight)

    class ToyConfig:
        architecture, model_type = "ToyMeanForCausalLM", "toy_mean"

        def __init__(self, raw):
            self.raw = raw

        @classmethod
        def from_hf_dict(cls, raw):
            return cls(raw)

        def to_hf_dict(self):
            return self.raw

    def toy_model_spec(cfg):
        hidden, raw = cfg.raw["hidden_size"], cfg.raw
        norm = lambda name: PartSpec("rmsnorm", {"dim": hidden, "eps": raw["eps"], "weight": name})
        layers = []
        for i in range(raw["layers"]):
            layers.append(LayerSpec(PartSpec("pre_norm", {
                "input_norm": norm("n1.weight"), "mixer": PartSpec("running_mean", {"hidden": hidden}),
                "post_norm": norm("n2.weight"),
                "feed_forward": PartSpec("gated_mlp", {"hidden": hidden, "inter": raw["inter"], "gate": "g.weight",
                                                       "up": "u.weight", "down": "d.weight"})}), f"blocks.{i}."))
        return ModelSpec("ToyMeanForCausalLM", raw["vocab_size"], hidden, 4096, "tok.weight", norm("final.weight"), None, layers)

    register_mixer("running_mean", RunningMean)
    register_architecture("ToyMeanForCausalLM", "toy_mean", ToyConfig, toy_model_spec)
    if own_kernel:
        build.register_source("toy_running_mean", ROOT / "tests" / "toy_kernels" / "running_mean.cu")
    try:
        raw = {"architectures": ["ToyMeanForCausalLM"], "model_type": "toy_mean", "vocab_size": 50, "hidden_size": 24,
               "inter": 40, "layers": 2, "eps": 1e-5}
        lb.write_model_folder(ToyConfig(raw), tmp_path, seed=3, std=0.3, norm_std=0.1, store_dtype=torch.float32)
        model = lb.load_model(tmp_path, device="cuda", dtype="fp32")       # the class is chosen by config.json
        if own_kernel:
            assert "toy_running_mean" in model.kernel_libraries(torch.float32)
            assert build.library_path("toy_running_mean").is_file()        # compiled when the model was built
        assert [n[1] for n in model.cache_needs()] == [StateNeed((25,), torch.float32)] * 2
        cache = lb.PagedKVCache(model, 4, block_tokens=4, max_requests=3)
        assert len(cache.paged) == 0 and cache.states[0].pool.shape == (2, 4, 25)
        step = StepFunction(model, cache)

        def plain(tokens):
            from safetensors.torch import load_file
            w = load_file(str(tmp_path / "model.safetensors"))
            x = w["tok.weight"][torch.tensor(tokens)]
            for i in range(2):
                p = f"blocks.{i}."
                h = plain_rmsnorm(x, w[p + "n1.weight"], 1e-5)
                mean = h.cumsum(0) / torch.arange(1, len(tokens) + 1)[:, None]
                x = x + mean @ w[p + "mean_proj.weight"].T
                x = x + plain_mlp(plain_rmsnorm(x, w[p + "n2.weight"], 1e-5), w[p + "g.weight"], w[p + "u.weight"], w[p + "d.weight"])
            return plain_rmsnorm(x, w["final.weight"], 1e-5) @ w["tok.weight"].T

        a_tokens, b_tokens = random_prompt(50, 23, 1), random_prompt(50, 9, 2)
        a, b = cache.open("a"), cache.open("b")
        got_a = [step([lb.StepEntry(a, a_tokens[:10], list(range(10)))])]
        # the rest of a in portions, b beside it: two requests' states in one batch
        both = step([lb.StepEntry(a, a_tokens[10:12], [0, 1]), lb.StepEntry(b, b_tokens, list(range(9)))])
        got_a.append(both[:2]); got_b = both[2:]
        for t in a_tokens[12:]:
            got_a.append(step([lb.StepEntry(a, [t], [0])]))
        expected_a, expected_b = plain(a_tokens), plain(b_tokens)
        assert (torch.cat(got_a).cpu() - expected_a).abs().max() <= tolerance(expected_a, torch.float32)
        assert (got_b.cpu() - expected_b).abs().max() <= tolerance(expected_b, torch.float32)
        cache.close(a)
        c = cache.open("c")                                       # a's slot again: the state starts from zero
        assert c.slot == a.slot
        got_c = step([lb.StepEntry(c, b_tokens, list(range(9)))])
        assert (got_c.cpu() - expected_b).abs().max() <= tolerance(expected_b, torch.float32)
    finally:
        unregister("mixer", "running_mean")
        unregister_architecture("ToyMeanForCausalLM")


def test_a_toy_position_encoding_and_a_toy_routed_feed_forward_run_in_the_same_blocks(tmp_path):
    """Two more parts defined here, not in the package, beside the package's attention and norms: a
    rotary encoding over positions divided by a factor, applied as a step of its own (it offers no
    table for the fused kernel), and a feed-forward that routes every token to one of three gated
    MLPs. Registered, built from a model folder, stepped whole, in portions and token by token."""
    from layover_b200.config import register_architecture, unregister_architecture
    from layover_b200.models import ModelSpec, LayerSpec
    from layover_b200.parts import Part, PartSpec, register_feed_forward, register_position, unregister
    from layover_b200.weights import TensorSpec
    from plain_qwen3 import plain_apply_rope, plain_attention, plain_linear, plain_rope_tables

    class ScaledRotary(Part):
        def __init__(self, params, prefix):
            super().__init__(params, prefix)
            self.dim, self.theta, self.factor = params["dim"], params["theta"], params["factor"]

        def tables(self, batch):
            return None                                   # not something the fused kernel can apply

        def apply(self, q, k, positions):
            inv = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2, dtype=torch.float32, device=q.device) / self.dim))
            angle = (positions.float() / self.factor)[:, None] * inv[None, :]
            cos, sin = torch.cat((angle, angle), -1).cos()[:, None, :], torch.cat((angle, angle), -1).sin()[:, None, :]
            for x in (q, k):
                if x is not None:
                    half = self.dim // 2
                    rotated = torch.cat((-x[..., half:], x[..., :half]), -1)
                    x.copy_(x * cos + rotated * sin)

    class Routed(Part):
        def __init__(self, params, prefix):
            super().__init__(params, prefix)
            self.hidden, self.inter, self.experts = params["hidden"], params["inter"], params["experts"]

        def names(self, e):
            return [f"{self.prefix}mlp.experts.{e}.{n}.weight" for n in ("gate", "up", "down")]

        def tensor_specs(self):
            specs = [TensorSpec(self.prefix + "mlp.router.weight", (self.experts, self.hidden), kind="keep32")]
            for e in range(self.experts):
                g, u, d = self.names(e)
                specs += [TensorSpec(g, (self.inter, self.hidden)), TensorSpec(u, (self.inter, self.hidden)),
                          TensorSpec(d, (self.hidden, self.inter))]
            return specs

        def bind(self, tensors, runtime):
            super().bind(tensors, runtime)
            self.router = tensors[self.prefix + "mlp.router.weight"]
            self.weights = [[tensors[n] for n in self.names(e)] for e in range(self.experts)]

        def forward(self, h):
            choice = (h.float() @ self.router.T).argmax(-1)          # router logits in 32-bit
            out = torch.zeros_like(h)
            for e, (gate, up, down) in enumerate(self.weights):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    x = h[rows].contiguous()
                    act = torch.nn.functional.silu(self.runtime.linear(x, gate)) * self.runtime.linear(x, up)
                    out[rows] = self.runtime.linear(act, down)
            return out

    class ToyConfig:
        architecture, model_type = "ToyRoutedForCausalLM", "toy_routed"

        def __init__(self, raw):
            self.raw = raw

        @classmethod
        def from_hf_dict(cls, raw):
            return cls(raw)

        def to_hf_dict(self):
            return self.raw

    def toy_model_spec(cfg):
        raw = cfg.raw
        hidden = raw["hidden_size"]
        norm = lambda name: PartSpec("rmsnorm", {"dim": hidden, "eps": raw["eps"], "weight": name})
        position = PartSpec("scaled_rotary", {"dim": raw["head_dim"], "theta": 5000.0, "factor": 4.0})
        layers = []
        for i in range(raw["layers"]):
            layers.append(LayerSpec(PartSpec("pre_norm", {
                "input_norm": norm("n1.weight"),
                "mixer": PartSpec("attention", {"hidden": hidden, "q_heads": raw["q_heads"], "kv_heads": raw["kv_heads"],
                                                "head_dim": raw["head_dim"], "qk_norm_eps": None, "position": position,
                                                "q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight",
                                                "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight"}),
                "post_norm": norm("n2.weight"),
                "feed_forward": PartSpec("routed", {"hidden": hidden, "inter": raw["inter"], "experts": 3})}), f"blocks.{i}."))
        return ModelSpec("ToyRoutedForCausalLM", raw["vocab_size"], hidden, 4096, "tok.weight", norm("final.weight"), None, layers)

    register_position("scaled_rotary", ScaledRotary)
    register_feed_forward("routed", Routed)
    register_architecture("ToyRoutedForCausalLM", "toy_routed", ToyConfig, toy_model_spec)
    try:
        raw = {"architectures": ["ToyRoutedForCausalLM"], "model_type": "toy_routed", "vocab_size": 60, "hidden_size": 40,
               "inter": 56, "layers": 2, "eps": 1e-5, "q_heads": 3, "kv_heads": 1, "head_dim": 16}
        lb.write_model_folder(ToyConfig(raw), tmp_path, seed=8, std=0.3, norm_std=0.1, store_dtype=torch.float32)
        model = lb.load_model(tmp_path, device="cuda", dtype="fp32")

        def plain(tokens):
            from safetensors.torch import load_file
            w = load_file(str(tmp_path / "model.safetensors"))
            x = w["tok.weight"][torch.tensor(tokens)]
            n = len(tokens)
            cos, sin = plain_rope_tables(torch.arange(n).float() / 4.0, 16, 5000.0, torch.float32)
            for i in range(2):
                p = f"blocks.{i}."
                h = plain_rmsnorm(x, w[p + "n1.weight"], 1e-5)
                q = plain_linear(h, w[p + "self_attn.q_proj.weight"]).view(n, 3, 16)
                k = plain_linear(h, w[p + "self_attn.k_proj.weight"]).view(n, 1, 16)
                v = plain_linear(h, w[p + "self_attn.v_proj.weight"]).view(n, 1, 16)
                q, k = plain_apply_rope(q, cos, sin), plain_apply_rope(k, cos, sin)
                x = x + plain_linear(plain_attention(q, k, v).reshape(n, -1), w[p + "self_attn.o_proj.weight"])
                h = plain_rmsnorm(x, w[p + "n2.weight"], 1e-5)
                choice = (h @ w[p + "mlp.router.weight"].T).argmax(-1)
                routed = torch.zeros_like(h)
                for e in range(3):
                    rows = choice == e
                    routed[rows] = plain_mlp(h[rows], *(w[f"{p}mlp.experts.{e}.{name}.weight"] for name in ("gate", "up", "down")))
                x = x + routed
            return plain_rmsnorm(x, w["final.weight"], 1e-5) @ w["tok.weight"].T

        tokens = random_prompt(60, 37, 5)
        expected = plain(tokens)
        for cuts in ([37], [5, 2, 16, 14], [20] + [1] * 17):
            got, cache, seq = step_in_portions(model, tokens, 4, cuts, blocks=16)
            assert (got - expected).abs().max() <= tolerance(expected, torch.float32), cuts
            cache.close(seq)
    finally:
        unregister("position", "scaled_rotary")
        unregister("feed_forward", "routed")
        unregister_architecture("ToyRoutedForCausalLM")

