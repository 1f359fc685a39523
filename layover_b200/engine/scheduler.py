"""Continuous batching with chunked prefill, above the step function.

Requests wait in arrival order, are admitted while a batch slot and a state slot are free and the
cache can hold their worst case, are fed their prompt in portions under a token budget beside the
running decodes, then decode one token a step until they finish; their pages and state slot go
back at once and the next waiting request may land on the same pages (layover/engine.py:75-232).

When pages run out: admission reserves every running request's worst-case growth (prompt plus
`max_new_tokens`), so a running request can never fail to get a page and nothing is ever
preempted or recomputed; a request that does not fit yet waits at the head of the queue (first
come, first served) and a request that could never fit is refused when it is added
(layover/engine.py:91-132). An `OutOfBlocks` that reaches `step()` is therefore a bug, not a
state.

The token budget of a step: with `max_batched_tokens` one number covers the whole step, the
decoding requests take one token each first and what is left goes to prompt portions in running
order, each at most `prefill_chunk` long. Without it the reference's rule holds: `prefill_budget`
prompt tokens a step, decoded tokens not counted (layover/engine.py:64-68,157-176).

What a request samples with (temperature, seed) is written into its record on the device when it
is admitted (`sampling.request_record`); every later step names the request's newest token as
"the one in its record" (`DEVICE_TOKEN`), so no token id travels back to the device.

Pipelined stepping (`step_pipelined`, used by `run_until_idle`): a step is launched before the
host has read the tokens of the step before it. Which requests decode next does not depend on
the token values (finishing by `max_new_tokens` is a count), so the host reads the previous
step's tokens while the GPU already runs the next step, and the scheduler, the batch building
and the copies cost no GPU time. A request that ends on a stop token is found out one step late:
it has one more step in flight, whose token is dropped. `step()` is the same step with the
tokens read at once.

Differences from the reference, on purpose: a step is ONE batch (prompt portions and decoded
tokens together) instead of one call per prefilling request followed by a decode call; the
first token of a request is sampled from the last row of its prompt and the request joins the
decodes in the next step (the reference also runs it through a decode in the same step,
layover/engine.py:172-174,220-223); sampling may use a temperature.
"""

from __future__ import annotations

import time
from collections import deque
from collections.abc import Callable
from dataclasses import dataclass, field
from enum import Enum

from ..sampling.sampler import SamplingParams, request_record
from .batch import DEVICE_TOKEN, StepEntry


class State(Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODE = "decode"
    FINISHED = "finished"


@dataclass
class Request:
    request_id: str
    prompt: list[int]
    max_new_tokens: int
    stop_tokens: frozenset[int] = frozenset()
    temperature: float = 0.0
    seed: int = 0
    ignore_eos: bool = False     # generate max_new_tokens whatever is sampled (layover/server.py:183,195)
    state: State = State.WAITING
    generated: list[int] = field(default_factory=list)
    prefilled: int = 0
    on_token: Callable[["Request", int], None] | None = None
    on_finish: Callable[["Request"], None] | None = None
    submitted_at: float = 0.0
    admitted_at: float | None = None
    first_token_at: float | None = None
    finished_at: float | None = None
    error: str | None = None
    cache: object = None   # the cache manager's record of this request while it runs
    pending: int = 0       # tokens sampled for it that the host has not read yet

    @property
    def max_tokens(self) -> int:
        return len(self.prompt) + self.max_new_tokens

    @property
    def done(self) -> bool:
        if len(self.generated) >= self.max_new_tokens:
            return True
        return bool(self.generated) and not self.ignore_eos and self.generated[-1] in self.stop_tokens


@dataclass(frozen=True)
class EngineConfig:
    max_batch: int = 32          # most requests running at a time
    prefill_chunk: int = 512     # most prompt tokens of one request in a step
    prefill_budget: int = 512    # most prompt tokens of all requests in a step (when the next is None)
    max_batched_tokens: int | None = None   # most tokens of a whole step: decoded tokens first, the rest for prompts

    def __post_init__(self):
        if self.max_batch < 1 or self.prefill_chunk < 1 or self.prefill_budget < 1:
            raise ValueError("max_batch, prefill_chunk and prefill_budget must be positive")
        if self.max_batched_tokens is not None and self.max_batched_tokens < self.max_batch:
            # with fewer, a batch full of decoding requests would leave no token for a prompt for ever
            raise ValueError(f"max_batched_tokens ({self.max_batched_tokens}) must be at least max_batch ({self.max_batch})")


class RequestTooLarge(ValueError):
    """The request could never fit in the KV pool or the model's positions."""


@dataclass
class _Launched:
    """A step whose tokens the host has not read yet."""
    sampled: list[Request]
    tokens: object               # its `result()` gives one token per sampled request


class Engine:
    def __init__(self, model, cache, config: EngineConfig = EngineConfig(),
                 clock: Callable[[], float] = time.monotonic, step_fn=None, cuda_graphs: bool = False):
        """`step_fn`: what runs a batch; by default a `StepFunction` over `model` and `cache`. It must
        offer `sample(entries)`, whose result's `result()` lists one token per entry that wants one, and
        `max_position`."""
        self.model, self.cache, self.config, self.clock = model, cache, config, clock
        if step_fn is None:
            from .step import StepFunction
            # a whole chunk of one prompt, alone in its step, is captured as well as the decode steps
            step_fn = StepFunction(model, cache, cuda_graphs=cuda_graphs,
                                   portion_graph_tokens=(config.prefill_chunk,) if cuda_graphs else ())
        self.step_fn = step_fn
        self.max_position = step_fn.max_position
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "largest_batch": 0, "dropped_tokens": 0}
        self._inflight: _Launched | None = None

    # ------------------------------------------------------------------ admission
    def add_request(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("prompt must not be empty")
        if request.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if request.temperature < 0:
            raise ValueError("temperature must not be negative")
        if request.max_tokens > self.max_position:
            raise RequestTooLarge(f"{request.request_id}: exceeds max_position_embeddings")
        for g, group in enumerate(self.cache.paged):
            if self._peak(g, request) > group.allocator.num_blocks:
                raise RequestTooLarge(f"{request.request_id}: larger than the KV pool")
        request.submitted_at = self.clock()
        self.waiting.append(request)

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    def _peak(self, group: int, request: Request) -> int:
        return self.cache.peak_blocks(group, request.max_tokens, self.config.prefill_chunk)

    def blocks_still_needed(self, request: Request) -> list[int]:
        """Per cache group, the most pages the request may still take before it finishes."""
        out = []
        for g in range(len(self.cache.paged)):
            held = 0
            if request.cache is not None:
                table = request.cache.tables[g]
                held = len(table.blocks) - table.first_live
            out.append(max(0, self._peak(g, request) - held))
        return out

    def available_blocks(self) -> list[int]:
        """Per cache group, free pages not spoken for by the requests already running."""
        reserved = [0] * len(self.cache.paged)
        for request in self.running:
            for g, need in enumerate(self.blocks_still_needed(request)):
                reserved[g] += need
        return [group.allocator.num_free - r for group, r in zip(self.cache.paged, reserved)]

    def _admit(self) -> None:
        """First come, first served: the head of the queue gets in when a batch place, a state slot and
        its worst case of pages in every group are free; nobody overtakes it."""
        while self.waiting and len(self.running) < self.config.max_batch and self.cache.num_free_slots > 0:
            head = self.waiting[0]
            if any(need > free for need, free in zip(self.blocks_still_needed(head), self.available_blocks())):
                return
            self.waiting.popleft()
            record = request_record(SamplingParams(head.temperature, head.seed), len(head.prompt))
            head.cache = self.cache.open(head.request_id, record)
            head.state = State.PREFILL
            head.admitted_at = self.clock()
            self.running.append(head)

    # ------------------------------------------------------------------ one step
    def plan(self) -> list[tuple[Request, list[int], bool]]:
        """This step's batch: (request, tokens, whether a token is sampled from its last row). Every
        decoding request that still has tokens to make takes part with its newest token; prompts
        share what the step's budget leaves."""
        plan = []
        for request in self.running:
            if request.state is not State.DECODE:
                continue
            if len(request.generated) + request.pending >= request.max_new_tokens:
                continue                                   # its last token is sampled, perhaps not read yet
            if request.done:
                continue                                   # ended on a stop token; leaves once nothing of it is in flight
            plan.append((request, [DEVICE_TOKEN], True))
        config = self.config
        if config.max_batched_tokens is None:
            budget = config.prefill_budget
        else:
            budget = config.max_batched_tokens - len(plan)      # decoded tokens first, the rest for prompts
        for request in self.running:
            if budget <= 0:
                break
            if request.state is not State.PREFILL:
                continue
            count = min(config.prefill_chunk, budget, len(request.prompt) - request.prefilled)
            tokens = request.prompt[request.prefilled: request.prefilled + count]
            budget -= count
            plan.append((request, tokens, request.prefilled + count == len(request.prompt)))
        return plan

    def _launch(self) -> _Launched | None:
        """Admit, plan and launch one step; the requests' counters move on, their tokens are pending."""
        self._admit()
        plan = self.plan()
        if not plan:
            return None
        entries = [StepEntry(request.cache, tokens, [len(tokens) - 1] if sample else []) for request, tokens, sample in plan]
        tokens = self.step_fn.sample(entries)
        sampled = []
        for request, fed, sample in plan:
            if request.state is State.PREFILL:
                request.prefilled += len(fed)
                self.stats["prefill_tokens"] += len(fed)
                if sample:
                    request.state = State.DECODE          # its first token is on its way
            else:
                self.stats["decode_tokens"] += 1
            if sample:
                request.pending += 1
                sampled.append(request)
        self.stats["steps"] += 1
        self.stats["largest_batch"] = max(self.stats["largest_batch"], len(plan))
        return _Launched(sampled, tokens)

    def _take_in(self, launched: _Launched) -> None:
        """Read a launched step's tokens and hand them to their requests."""
        for request, token in zip(launched.sampled, launched.tokens.result()):
            request.pending -= 1
            if request.done or request.state is State.FINISHED:   # ended on a stop token one step earlier
                self.stats["dropped_tokens"] += 1
                continue
            token = int(token)
            request.generated.append(token)
            if request.first_token_at is None:
                request.first_token_at = self.clock()
            if request.on_token is not None:
                request.on_token(request, token)

    def _retire(self) -> bool:
        """Requests that are done leave: pages and slot go back, `on_finish` is told."""
        leaving = [r for r in self.running if r.state is State.DECODE and r.pending == 0 and r.done]
        if not leaving:
            return False
        gone = {id(r) for r in leaving}
        self.running = [r for r in self.running if id(r) not in gone]
        for request in leaving:
            self.cache.close(request.cache)
            request.cache, request.state, request.finished_at = None, State.FINISHED, self.clock()
            self.finished.append(request)
            if request.on_finish is not None:
                request.on_finish(request)
        return True

    def step(self) -> bool:
        """Advance every runnable request once and read its token. Returns whether anything happened."""
        if self._inflight is not None:                 # a pipelined step is still out: take it in first
            self._take_in(self._inflight)
            self._inflight = None
            self._retire()
        launched = self._launch()
        if launched is not None:
            self._take_in(launched)
        retired = self._retire()
        return launched is not None or retired

    def step_pipelined(self) -> bool:
        """Launch the next step, then take in the tokens of the step before it."""
        previous = self._inflight
        self._inflight = self._launch()
        retired = False
        if previous is not None:
            self._take_in(previous)
            retired = self._retire()
        return self._inflight is not None or previous is not None or retired

    def run_until_idle(self, max_steps: int = 1_000_000) -> list[Request]:
        """Step (pipelined) until nothing waits, runs or is in flight; the finished requests."""
        steps = 0
        while not (self.idle and self._inflight is None):
            if steps >= max_steps:
                raise RuntimeError("engine did not become idle")
            steps += 1
            if not self.step_pipelined() and self.waiting and not self.running:
                raise RuntimeError("the head request can never be admitted")
        return self.finished
