"""The scheduler's decisions on the CPU, with a step function that computes nothing: admission,
portions under the token budget, decoding, finishing and freeing, and what happens when pages run
out (layover's own behaviour tests are tests/test_engine.py:127-208 there)."""

import random

import pytest
import torch

from layover_b200.cache import CacheManager, OutOfBlocks
from layover_b200.engine import Engine, EngineConfig, Request, RequestTooLarge, State
from layover_b200.parts.base import PagedKVNeed


class FakeTokens:
    def __init__(self, values):
        self.values = values

    def result(self):
        return list(self.values)


class FakeStep:
    """Counts tokens into the cache like the real step function; the 'token' it samples for a
    request is the request's length so far, which makes the emitted tokens easy to predict."""

    max_position = 4096

    def __init__(self, cache):
        self.cache = cache
        self.batches = []
        self.read_back = 0

    def sample(self, entries):
        for e in entries:
            self.cache.grow(e.seq, e.seq.num_tokens + len(e.tokens))    # must never raise under the scheduler
        self.batches.append([(e.seq.request_id, len(e.tokens), list(e.want)) for e in entries])
        tokens = []
        for e in entries:
            self.cache.commit(e.seq, e.seq.num_tokens + len(e.tokens))
            tokens += [e.seq.num_tokens] * len(e.want)
        return FakeTokens(tokens)


def make(blocks=64, page=4, config=EngineConfig(), window=None, max_requests=8):
    cache = CacheManager([(0, PagedKVNeed(1, 16, window), None)], blocks, page, torch.float32, None, max_requests)
    clock = iter(range(10**6))
    engine = Engine(None, cache, config, clock=lambda: next(clock), step_fn=FakeStep(cache))
    return engine, cache


def test_portions_respect_chunk_and_budget_and_mix_with_decodes():
    engine, cache = make(config=EngineConfig(max_batch=4, prefill_chunk=8, prefill_budget=12))
    engine.add_request(Request("short", [1] * 3, 6))
    engine.add_request(Request("long", [2] * 30, 2))
    engine.step()
    assert engine.step_fn.batches[0] == [("short", 3, [2]), ("long", 8, [])]       # chunk caps one request
    engine.step()
    assert engine.step_fn.batches[1] == [("short", 1, [0]), ("long", 8, [])]       # decode beside a portion
    engine.run_until_idle()
    sizes = [n for batch in engine.step_fn.batches for name, n, _ in batch if name == "long" and n > 1]
    assert sizes == [8, 8, 8, 6] and sum(sizes) == 30
    short = next(r for r in engine.finished if r.request_id == "short")
    assert short.generated == [3, 4, 5, 6, 7, 8]                                     # a token every step: never stalled
    assert all(r.state is State.FINISHED for r in engine.finished)
    assert cache.num_free == 64
    cache.check()


def test_budget_is_shared_between_prompts():
    engine, _ = make(config=EngineConfig(max_batch=4, prefill_chunk=100, prefill_budget=10))
    engine.add_request(Request("a", [1] * 7, 1))
    engine.add_request(Request("b", [1] * 7, 1))
    engine.step()
    assert engine.step_fn.batches[0] == [("a", 7, [6]), ("b", 3, [])]
    engine.step()
    assert engine.step_fn.batches[1] == [("b", 4, [3])]


def test_admission_waits_for_pages_and_reuses_them():
    engine, cache = make(blocks=4, page=16)                     # as the reference's 4-block pool test
    for name in ("first", "second"):
        engine.add_request(Request(name, [1] * 40, 8))          # 48 tokens = 3 pages each
    engine.step()
    assert [r.request_id for r in engine.running] == ["first"] and len(engine.waiting) == 1
    finished = engine.run_until_idle()
    assert [r.request_id for r in finished] == ["first", "second"]
    assert finished[1].admitted_at > finished[0].finished_at - 1
    assert cache.num_free == 4
    cache.check()


def test_head_of_line_is_not_overtaken():
    engine, _ = make(blocks=4, page=16)
    engine.add_request(Request("big", [1] * 40, 8))
    engine.add_request(Request("big2", [1] * 40, 8))
    engine.add_request(Request("small", [1] * 2, 2))             # would fit beside "big", but waits its turn
    engine.step()
    assert [r.request_id for r in engine.running] == ["big"]
    assert [r.request_id for r in engine.waiting] == ["big2", "small"]


def test_running_requests_never_run_out_of_pages():
    rng = random.Random(0)
    engine, cache = make(blocks=9, page=4, config=EngineConfig(max_batch=5, prefill_chunk=6, prefill_budget=9))
    for i in range(40):
        engine.add_request(Request(f"r{i}", [1] * rng.randint(1, 20), rng.randint(1, 12)))
    steps = 0
    while not engine.idle:
        engine.step()          # FakeStep.grow would raise OutOfBlocks if the reservation were wrong
        cache.check()
        steps += 1
        assert steps < 5000
    assert len(engine.finished) == 40 and cache.num_free == 9
    assert engine.stats["largest_batch"] > 1


def test_max_batch_limits_running_requests():
    engine, _ = make(config=EngineConfig(max_batch=2, prefill_chunk=64, prefill_budget=64))
    for i in range(5):
        engine.add_request(Request(str(i), [1, 2], 3))
    engine.step()
    assert len(engine.running) == 2 and len(engine.waiting) == 3
    engine.run_until_idle()
    assert len(engine.finished) == 5


def test_stop_token_and_limits():
    engine, cache = make()
    engine.add_request(Request("s", [9] * 5, 50, stop_tokens=frozenset({7})))
    engine.run_until_idle()
    assert engine.finished[0].generated == [5, 6, 7]            # stops on the stop token, which is kept
    assert cache.num_free == 64
    with pytest.raises(ValueError, match="empty"):
        engine.add_request(Request("e", [], 4))
    with pytest.raises(RequestTooLarge, match="max_position"):
        engine.add_request(Request("p", [1] * 4000, 200))
    small, _ = make(blocks=2, page=4)
    with pytest.raises(RequestTooLarge, match="KV pool"):
        small.add_request(Request("k", [1] * 8, 4))


def test_last_token_is_never_fed_and_timestamps_are_ordered():
    engine, _ = make()
    seen = []
    engine.add_request(Request("t", [1, 2, 3], 4, on_token=lambda r, t: seen.append(t),
                               on_finish=lambda r: seen.append("end")))
    engine.run_until_idle()
    request = engine.finished[0]
    fed = sum(n for batch in engine.step_fn.batches for _, n, _ in batch)
    assert fed == 3 + 3                                          # the prompt and all generated tokens but the last
    assert seen == [3, 4, 5, 6, "end"]
    assert request.submitted_at <= request.admitted_at <= request.first_token_at <= request.finished_at


def test_each_requests_sampling_parameters_go_into_its_record_at_admission():
    import struct

    from layover_b200 import ops

    engine, cache = make()
    opened = []
    real_open = cache.open
    cache.open = lambda rid, record=None: (opened.append((rid, record)), real_open(rid, record))[1]
    engine.add_request(Request("a", [1, 1], 3, temperature=0.5, seed=(7 << 32) | 0xFFFFFFFE))
    engine.add_request(Request("b", [1], 2))
    engine.run_until_idle()
    (name_a, rec_a), (name_b, rec_b) = opened
    assert (name_a, name_b) == ("a", "b") and len(rec_a) == ops.RECORD_WORDS
    assert struct.unpack("<f", struct.pack("<i", rec_a[ops.RECORD_TEMPERATURE]))[0] == 0.5
    assert rec_a[ops.RECORD_SEED_LO] == -2 and rec_a[ops.RECORD_SEED_HI] == 7       # the 64-bit seed as two words
    assert rec_a[ops.RECORD_COUNT] == 0 and rec_a[ops.RECORD_POSITION] == 2
    assert rec_b[ops.RECORD_TEMPERATURE] == 0 and rec_b[ops.RECORD_SEED_LO] == 0
    with pytest.raises(ValueError, match="temperature"):
        engine.add_request(Request("c", [1], 2, temperature=-1.0))


def test_decoded_tokens_are_named_not_sent():
    """A decoding request's newest token stays on the device: the step names it, no id travels."""
    from layover_b200.engine.batch import DEVICE_TOKEN

    engine, cache = make()
    seen = []
    real = engine.step_fn.sample
    engine.step_fn.sample = lambda entries: (seen.append([list(e.tokens) for e in entries]), real(entries))[1]
    engine.add_request(Request("a", [5, 6, 7], 3))
    engine.run_until_idle()
    assert seen == [[[5, 6, 7]], [[DEVICE_TOKEN]], [[DEVICE_TOKEN]]]


def test_one_budget_for_the_whole_step_counts_decoded_tokens_first():
    config = EngineConfig(max_batch=4, prefill_chunk=8, max_batched_tokens=10)
    engine, _ = make(config=config)
    engine.add_request(Request("d1", [1] * 2, 9))
    engine.add_request(Request("d2", [1] * 2, 9))
    engine.step()                                                   # both prompts whole: 4 tokens of 10
    engine.add_request(Request("long", [2] * 30, 2))
    engine.add_request(Request("long2", [2] * 30, 2))
    engine.step()
    # two decoded tokens first, then 8 prompt tokens (the chunk would allow 8, the rest is 8), none left for long2
    assert engine.step_fn.batches[1] == [("d1", 1, [0]), ("d2", 1, [0]), ("long", 8, [])]
    engine.step()
    assert sum(n for _, n, _ in engine.step_fn.batches[2]) == 10
    with pytest.raises(ValueError, match="max_batched_tokens"):
        EngineConfig(max_batch=8, max_batched_tokens=4)
    # without it the reference's rule: prefill_budget prompt tokens, decoded tokens not counted
    engine, _ = make(config=EngineConfig(max_batch=4, prefill_chunk=8, prefill_budget=8))
    engine.add_request(Request("d1", [1] * 2, 9))
    engine.step()
    engine.add_request(Request("long", [2] * 30, 2))
    engine.step()
    assert engine.step_fn.batches[1] == [("d1", 1, [0]), ("long", 8, [])]


def test_ignore_eos_generates_to_the_limit():
    engine, _ = make()
    engine.add_request(Request("s", [9] * 5, 6, stop_tokens=frozenset({7}), ignore_eos=True))
    engine.add_request(Request("t", [9] * 5, 6, stop_tokens=frozenset({7})))
    engine.run_until_idle()
    by_name = {r.request_id: r.generated for r in engine.finished}
    assert by_name["s"] == [5, 6, 7, 8, 9, 10] and by_name["t"] == [5, 6, 7]


def test_admission_counts_a_free_state_slot():
    """More batch places than state slots: the third request waits for a slot, nothing raises."""
    engine, cache = make(config=EngineConfig(max_batch=4, prefill_chunk=64, prefill_budget=64), max_requests=2)
    for i in range(3):
        engine.add_request(Request(str(i), [1, 2], 3))
    engine.step()
    assert len(engine.running) == 2 and len(engine.waiting) == 1 and cache.num_free_slots == 0
    engine.run_until_idle()
    assert len(engine.finished) == 3 and cache.num_free_slots == 2
    cache.check()


def test_a_stop_token_found_a_step_late_drops_the_token_in_flight():
    engine, cache = make()
    engine.add_request(Request("s", [9] * 5, 50, stop_tokens=frozenset({7})))
    engine.add_request(Request("u", [9] * 2, 8))
    engine.run_until_idle()                                         # pipelined
    by_name = {r.request_id: r.generated for r in engine.finished}
    assert by_name["s"] == [5, 6, 7] and by_name["u"] == list(range(2, 10))
    assert engine.stats["dropped_tokens"] == 1 and cache.num_free == 64
    cache.check()


def test_a_window_lets_long_requests_fit_a_small_pool():
    engine, cache = make(blocks=6, page=4, window=8, config=EngineConfig(max_batch=2, prefill_chunk=4, prefill_budget=4))
    engine.add_request(Request("w", [1] * 50, 30))               # 80 tokens = 20 pages without the window
    engine.run_until_idle()
    assert len(engine.finished[0].generated) == 30 and cache.num_free == 6


def test_out_of_blocks_from_a_step_is_an_error_not_a_state():
    engine, cache = make(blocks=3, page=4)
    engine.add_request(Request("x", [1] * 4, 4))
    thief = cache.open("thief")
    engine.step()
    cache.grow(thief, 8)                                         # someone takes pages behind the scheduler's back
    with pytest.raises(OutOfBlocks):
        for _ in range(10):
            engine.step()
