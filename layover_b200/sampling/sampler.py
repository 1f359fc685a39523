"""Choosing the next token of each request from its logits, on the device.

Greedy is the first index of the maximum, as the reference's `argmax` (layover/engine.py:139-141,
187). The reference takes `temperature` in its API and ignores it (layover/server.py:13-14); here
a temperature T > 0 draws from softmax(logits / T) with the Gumbel-max rule and a counter-based
generator keyed by the request's seed and the number of tokens it has sampled so far, so a
request's tokens are the same whatever else is in the batch.

What a request samples with lives in its record on the device (`CacheManager.records`, one row of
int32 words per state slot): `request_record` makes the row that is written when the request is
admitted, and from then on the sampling kernel reads seed, counter and temperature there, writes
the chosen token back as the request's last token and bumps the counter. A step uploads nothing
for sampling, the next step's embedding reads the last token straight from the record, and the
sampling launch sits inside a captured decode step like any other kernel.
"""

from __future__ import annotations

import struct
from dataclasses import dataclass

import torch

from .. import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0


def _signed(word: int) -> int:
    return word - (1 << 32) if word >= (1 << 31) else word


def request_record(params: SamplingParams = SamplingParams(), prompt_tokens: int = 0) -> list[int]:
    """The int32 words of a new request's record (layout: `ops.RECORD_*`)."""
    if params.temperature < 0:
        raise ValueError("temperature must not be negative")
    words = [0] * ops.RECORD_WORDS
    words[ops.RECORD_POSITION] = int(prompt_tokens)
    words[ops.RECORD_SEED_LO] = _signed(params.seed & 0xFFFFFFFF)
    words[ops.RECORD_SEED_HI] = _signed((params.seed >> 32) & 0xFFFFFFFF)
    words[ops.RECORD_COUNT] = 0
    words[ops.RECORD_TEMPERATURE] = struct.unpack("<i", struct.pack("<f", float(params.temperature)))[0]
    words[ops.RECORD_LAST_TOKEN] = 0
    return words


class Sampler:
    """Launches the sampling kernel over a step's wanted rows.

    `records`: the cache manager's per-request records. `status_libraries`: kernel libraries whose
    error words travel to the host behind the tokens (see `ops.status_words`)."""

    def __init__(self, device: torch.device | str, records: torch.Tensor | None, status_libraries=()):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ops.KernelError("the sampler runs on a CUDA device only")
        self.records = records
        self.status, self.status_names = ops.status_words(self.device, tuple(status_libraries))
        self.n_status = 0 if self.status is None else self.status.shape[0]
        self._host_ring: list[torch.Tensor] = []
        self._turn = 0

    def sample_into(self, logits: torch.Tensor, batch, tokens: torch.Tensor) -> torch.Tensor:
        """The kernel launch alone (what a captured graph holds): tokens[r] for every row of logits,
        then the status words."""
        use_records = self.records is not None
        return ops.sample(logits, tokens, self.records if use_records else None, batch.row_slots if use_records else None,
                          batch.positions if use_records else None, batch.logit_rows if use_records else None,
                          self.status)

    def launch(self, logits: torch.Tensor, batch) -> "PendingTokens":
        """Sample without waiting: the tokens stay on the device, in the requests' records, where the
        next step reads them, and travel to pinned host memory behind the kernel."""
        rows = logits.shape[0]
        if rows == 0:
            return PendingTokens(None, None, 0, 0, self)
        tokens = torch.empty(rows + self.n_status, dtype=torch.int32, device=self.device)
        self.sample_into(logits, batch, tokens)
        return self.collect(tokens, rows, rows)

    def collect(self, tokens: torch.Tensor, rows: int, sampled_rows: int) -> "PendingTokens":
        """Start the copy to the host of what `sample_into` wrote for `sampled_rows` rows of logits (the
        tokens, then the status words); the first `rows` of the tokens are the caller's."""
        count = sampled_rows + self.n_status
        if len(self._host_ring) < 4:
            self._host_ring.append(torch.empty(max(count, 256), dtype=torch.int32, pin_memory=True))
        index = self._turn % len(self._host_ring)
        self._turn += 1
        if self._host_ring[index].numel() < count:
            self._host_ring[index] = torch.empty(2 * count, dtype=torch.int32, pin_memory=True)
        host = self._host_ring[index][:count]
        host.copy_(tokens[:count], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(host, event, rows, sampled_rows, self)

    def explain(self, codes: list[int]) -> str:
        return ", ".join(f"{name}: code {code}" for name, code in zip(self.status_names, codes) if code)


class PendingTokens:
    """Sampled tokens on their way to the host. At most four may be outstanding per sampler (their
    pinned buffers are a ring of four)."""

    def __init__(self, host, event, rows: int, sampled_rows: int, sampler: Sampler):
        self._host, self._event, self._rows, self._sampled, self._sampler = host, event, rows, sampled_rows, sampler

    def result(self) -> list[int]:
        """The tokens, one per sampled row. Raises `ops.KernelError` if a kernel of this step reported a
        wait that ran out (its results cannot be trusted); the device's split counters and the error
        words are put back first, so that the next step runs on a clean state."""
        if self._host is None:
            return []
        self._event.synchronize()
        values = self._host.tolist()
        codes = values[self._sampled:]
        if any(codes):
            message = self._sampler.explain(codes)
            ops.reset_after_error(self._sampler.device)
            raise ops.KernelError(f"a kernel gave up waiting ({message}); this step's tokens are dropped")
        return values[: self._rows]
