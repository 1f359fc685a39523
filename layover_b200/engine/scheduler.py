"""Continuous batching with chunked prefill, above the step function.

Requests wait in arrival order, are admitted while a batch slot is free and the cache can hold
their worst case, are fed their prompt in portions under a token budget beside the running
decodes, then decode one token a step until they finish; their pages and state slot go back at
once and the next waiting request may land on the same pages (layover/engine.py:75-232).

When pages run out: admission reserves every running request's worst-case growth (prompt plus
`max_new_tokens`), so a running request can never fail to get a page and nothing is ever
preempted or recomputed; a request that does not fit yet waits at the head of the queue (first
come, first served) and a request that could never fit is refused when it is added
(layover/engine.py:91-132). An `OutOfBlocks` that reaches `step()` is therefore a bug, not a
state.

Pipelined stepping (`step_pipelined`, used by `run_until_idle` with the real sampler): a step is
launched before the host has read the tokens of the step before it. Which requests decode next
does not depend on the token values (finishing by `max_new_tokens` is a count), only the token
ids do, and those the next step reads on the device, straight from the sampler's output. The
host then reads the previous step's tokens while the GPU already runs the next step, so the
scheduler, the batch building and the copies cost no GPU time. A request that ends on a stop
token is found out one step late: it has one more step in flight, whose token is dropped.

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

from ..sampling.sampler import SamplingParams
from .batch import StepEntry


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
    pending: int = 0       # tokens sampled for it that the host has not read yet (pipelined stepping)

    @property
    def max_tokens(self) -> int:
        return len(self.prompt) + self.max_new_tokens

    @property
    def done(self) -> bool:
        if len(self.generated) >= self.max_new_tokens:
            return True
        return bool(self.generated) and self.generated[-1] in self.stop_tokens


@dataclass(frozen=True)
class EngineConfig:
    max_batch: int = 32          # most requests running at a time
    prefill_chunk: int = 512     # most prompt tokens of one request in a step
    prefill_budget: int = 512    # most prompt tokens of all requests in a step


class RequestTooLarge(ValueError):
    """The request could never fit in the KV pool or the model's positions."""


class Engine:
    def __init__(self, model, cache, config: EngineConfig = EngineConfig(),
                 clock: Callable[[], float] = time.monotonic, step_fn=None, sampler=None,
                 cuda_graphs: bool = False):
        self.model, self.cache, self.config, self.clock = model, cache, config, clock
        if step_fn is None:
            from .step import StepFunction
            step_fn = StepFunction(model, cache, cuda_graphs=cuda_graphs)
        if sampler is None:
            from ..sampling.sampler import Sampler
            sampler = Sampler(model.device)
        self.step_fn, self.sampler = step_fn, sampler
        self.max_position = step_fn.max_position
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "largest_batch": 0, "dropped_tokens": 0}
        self._inflight = None      # (requests sampled by the step in flight, its PendingTokens)

    # ------------------------------------------------------------------ admission
    def add_request(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("prompt must not be empty")
        if request.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
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
        while self.waiting and len(self.running) < self.config.max_batch:
            request = self.waiting[0]
            need, free = self.blocks_still_needed(request), self.available_blocks()
            if any(n > f for n, f in zip(need, free)):
                return  # head of the line waits; nobody overtakes it
            self.waiting.popleft()
            request.cache = self.cache.open(request.request_id)
            request.state = State.PREFILL
            request.admitted_at = self.clock()
            self.running.append(request)

    # ------------------------------------------------------------------ one step
    def plan(self) -> list[tuple[Request, list[int], bool]]:
        """This step's batch: (request, tokens, whether a token is sampled from its last row)."""
        plan = []
        for request in self.running:
            if request.state is State.DECODE and not request.done:
                plan.append((request, [request.generated[-1]], True))
        budget = self.config.prefill_budget
        for request in self.running:
            if request.state is not State.PREFILL or budget <= 0:
                continue
            count = min(self.config.prefill_chunk, budget, len(request.prompt) - request.prefilled)
            tokens = request.prompt[request.prefilled: request.prefilled + count]
            budget -= count
            plan.append((request, tokens, request.prefilled + count == len(request.prompt)))
        return plan

    def step(self) -> bool:
        """Advance every runnable request once. Returns whether anything happened."""
        self._admit()
        plan = self.plan()
        if plan:
            entries = [StepEntry(r.cache, tokens, [len(tokens) - 1] if sample else []) for r, tokens, sample in plan]
            logits = self.step_fn(entries)
            sampled = [r for r, _, sample in plan if sample]
            tokens = self.sampler(logits, [SamplingParams(r.temperature, r.seed) for r in sampled],
                                  [len(r.generated) for r in sampled])
            for request, new_tokens, _ in plan:
                if request.state is State.PREFILL:
                    request.prefilled += len(new_tokens)
                    self.stats["prefill_tokens"] += len(new_tokens)
                else:
                    self.stats["decode_tokens"] += 1
            for request, token in zip(sampled, tokens):
                self._emit(request, int(token))
            self.stats["steps"] += 1
            self.stats["largest_batch"] = max(self.stats["largest_batch"], len(plan))
        retired = self._retire()
        return bool(plan) or retired

    def _emit(self, request: Request, token: int) -> None:
        if request.state is State.PREFILL:
            request.state = State.DECODE
        request.generated.append(token)
        if request.first_token_at is None:
            request.first_token_at = self.clock()
        if request.on_token is not None:
            request.on_token(request, token)

    def _retire(self) -> bool:
        still_running, retired = [], False
        for request in self.running:
            if request.state is State.DECODE and request.done:
                request.state = State.FINISHED
                request.finished_at = self.clock()
                self.cache.close(request.cache)
                request.cache = None
                self.finished.append(request)
                if request.on_finish is not None:
                    request.on_finish(request)
                retired = True
            else:
                still_running.append(request)
        self.running = still_running
        return retired

    # ------------------------------------------------------------------ pipelined stepping
    def step_pipelined(self) -> bool:
        """Launch the next step, then take in the tokens of the step before it."""
        self._admit()
        previous = self._inflight
        source = {id(r): row for row, r in enumerate(previous[0])} if previous else {}
        plan = []
        for request in self.running:
            if request.state is State.DECODE and len(request.generated) + request.pending < request.max_new_tokens \
                    and not (request.pending == 0 and request.done):
                # its newest token: still on the device (row of the step in flight) or already here
                token = -(source[id(request)] + 1) if request.pending else request.generated[-1]
                plan.append((request, [token], True))
        budget = self.config.prefill_budget
        for request in self.running:
            if request.state is not State.PREFILL or budget <= 0:
                continue
            count = min(self.config.prefill_chunk, budget, len(request.prompt) - request.prefilled)
            tokens = request.prompt[request.prefilled: request.prefilled + count]
            budget -= count
            plan.append((request, tokens, request.prefilled + count == len(request.prompt)))
        launched = None
        if plan:
            entries = [StepEntry(r.cache, tokens, [len(tokens) - 1] if sample else []) for r, tokens, sample in plan]
            logits = self.step_fn(entries, previous[1].device if previous else None)
            sampled = [r for r, _, sample in plan if sample]
            pending = self.sampler.launch(logits, [SamplingParams(r.temperature, r.seed) for r in sampled],
                                          [len(r.generated) + r.pending for r in sampled])
            for request, new_tokens, _ in plan:
                if request.state is State.PREFILL:
                    request.prefilled += len(new_tokens)
                    self.stats["prefill_tokens"] += len(new_tokens)
                    if request.prefilled == len(request.prompt):
                        request.state = State.DECODE          # its first token is on its way
                else:
                    self.stats["decode_tokens"] += 1
            for request in sampled:
                request.pending += 1
            launched = (sampled, pending)
            self.stats["steps"] += 1
            self.stats["largest_batch"] = max(self.stats["largest_batch"], len(plan))
        retired = False
        if previous is not None:
            retired = self._take_in(previous)
        self._inflight = launched
        return bool(plan) or retired or previous is not None

    def _take_in(self, step) -> bool:
        """Read a launched step's tokens and hand them to their requests."""
        sampled, pending = step
        for request, token in zip(sampled, pending.result()):
            request.pending -= 1
            if request.state is State.FINISHED:        # ended on a stop token one step earlier
                self.stats["dropped_tokens"] += 1
                continue
            request.generated.append(int(token))
            if request.first_token_at is None:
                request.first_token_at = self.clock()
            if request.on_token is not None:
                request.on_token(request, int(token))
        return self._retire()

    def run_until_idle(self, max_steps: int = 1_000_000) -> list[Request]:
        pipelined = hasattr(self.sampler, "launch")
        for _ in range(max_steps):
            if self.idle and self._inflight is None:
                return self.finished
            progressed = self.step_pipelined() if pipelined else self.step()
            if not progressed and self.waiting and not self.running:
                raise RuntimeError("the head request can never be admitted")
        raise RuntimeError("engine did not become idle")
