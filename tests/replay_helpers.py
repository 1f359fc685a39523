"""Traces for the replay program in the ways a prompt can be cut, and a runner that feeds them
through `layover_b200.replay.trace.run` in this process."""

from __future__ import annotations

import json
from pathlib import Path
from types import SimpleNamespace

import numpy as np


def whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone, all of it in one step."""
    return [{"step": i, "entries": [{"id": name, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [name]}
            for i, (name, tokens) in enumerate(requests.items())]


def tail_decoded(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of each request in one step, the last `tail` tokens one by one."""
    steps = []
    for name, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"entries": [{"id": name, "tokens": tokens[:head], "want": list(range(head))}], "end": []})
        for at in range(head, len(tokens)):
            steps.append({"entries": [{"id": name, "tokens": [tokens[at]], "want": [0]}], "end": []})
        steps[-1]["end"] = [name]
    return number(steps)


def portions(requests: dict[str, list[int]], sizes=(2, 7, 3, 16, 2, 33, 5, 1, 64, 2)) -> list[dict]:
    """Each request alone in portions of changing size, down to two tokens."""
    steps = []
    for index, (name, tokens) in enumerate(requests.items()):
        at, turn = 0, index
        while at < len(tokens):
            size = min(sizes[turn % len(sizes)], len(tokens) - at)
            steps.append({"entries": [{"id": name, "tokens": tokens[at:at + size], "want": list(range(size))}], "end": []})
            at += size
            turn += 1
        steps[-1]["end"] = [name]
    return number(steps)


def mixed(requests: dict[str, list[int]], live_limit: int = 4, prompt_part: float = 0.6,
          sizes=(5, 2, 9, 3, 17, 2)) -> list[dict]:
    """Up to `live_limit` requests at a time: the first `prompt_part` of each goes in portions, the
    rest token by token, portions of some beside single tokens of others; a request that ends
    makes room for the next, which then lands on the pages it gave back."""
    waiting = list(requests.items())
    live: list[dict] = []
    steps, turn = [], 0
    while waiting or live:
        while waiting and len(live) < live_limit:
            name, tokens = waiting.pop(0)
            live.append({"id": name, "tokens": tokens, "at": 0, "prompt": max(1, int(len(tokens) * prompt_part))})
        entries, ended = [], []
        for slot, item in enumerate(live):
            if (turn + slot) % 5 == 4 and len(live) > 1:
                continue                                  # left out of this step; goes on later
            if item["at"] < item["prompt"]:
                size = min(sizes[(turn + slot) % len(sizes)], item["prompt"] - item["at"])
            else:
                size = 1
            part = item["tokens"][item["at"]:item["at"] + size]
            entries.append({"id": item["id"], "tokens": part, "want": list(range(len(part)))})
            item["at"] += len(part)
            if item["at"] == len(item["tokens"]):
                ended.append(item["id"])
        live = [item for item in live if item["id"] not in ended]
        if entries:
            steps.append({"entries": entries, "end": ended})
        turn += 1
    return number(steps)


def crowd(requests: dict[str, list[int]], decoded: int = 6, prompts_per_step: int = 16) -> list[dict]:
    """Many requests at once: the prompts (all but the last `decoded` tokens of each) go in, several
    whole prompts a step, then ALL requests decode together, one token each a step. Requests whose
    tokens run out drop out of the later steps, so the number of rows also takes values that are no
    bucket size."""
    names = list(requests)
    steps = []
    for at in range(0, len(names), prompts_per_step):
        entries = []
        for name in names[at:at + prompts_per_step]:
            head = max(1, len(requests[name]) - decoded)
            entries.append({"id": name, "tokens": requests[name][:head], "want": list(range(head))})
        steps.append({"entries": entries, "end": []})
    done = {name: max(1, len(requests[name]) - decoded) for name in names}
    while any(done[name] < len(requests[name]) for name in names):
        entries, ended = [], []
        for name in names:
            if done[name] < len(requests[name]):
                entries.append({"id": name, "tokens": [requests[name][done[name]]], "want": [0]})
                done[name] += 1
                if done[name] == len(requests[name]):
                    ended.append(name)
        steps.append({"entries": entries, "end": ended})
    return number(steps)


def number(steps: list[dict]) -> list[dict]:
    for index, step in enumerate(steps):
        step["step"] = index
    return steps


def max_live_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The --max-tokens a trace needs: the most tokens live requests hold, each rounded up."""
    held: dict[str, int] = {}
    most = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        most = max(most, sum(-(-n // round_to) * round_to for n in held.values()))
        for name in step["end"]:
            held.pop(name, None)
    return most


def run_trace(folder, dtype: str, steps: list[dict], out: Path, max_tokens: int | None = None, block_tokens: int = 16,
              cuda_graphs: bool = False, max_requests: int = 8):
    """Feed `steps` through the replay program's own loop; returns {request: {position: logits row}}."""
    from layover_b200.replay.trace import run

    args = SimpleNamespace(model=str(folder), dtype=dtype, out=str(out), block_tokens=block_tokens,
                           max_requests=max_requests, cuda_graphs=cuda_graphs,
                           max_tokens=max_tokens if max_tokens is not None else max_live_tokens(steps))
    said = []
    assert run(args, [json.dumps(s) for s in steps], say=lambda text, flush=True: said.append(text)) == 0
    assert said == [f"done {s['step']}" for s in steps]
    return collect(steps, out)


def collect(steps: list[dict], out: Path) -> dict[str, dict[int, np.ndarray]]:
    rows: dict[str, dict[int, np.ndarray]] = {}
    position: dict[str, int] = {}
    for step in steps:
        wanted = sum(len(e["want"]) for e in step["entries"])
        path = Path(out) / f"{step['step']}.f32"
        if wanted == 0:
            assert not path.exists()
            data = None
        else:
            data = np.fromfile(path, dtype="<f4").reshape(wanted, -1)
        at = 0
        for entry in step["entries"]:
            start = position.get(entry["id"], 0)
            for w in entry["want"]:
                rows.setdefault(entry["id"], {})[start + w] = data[at]
                at += 1
            position[entry["id"]] = start + len(entry["tokens"])
        for name in step["end"]:
            position.pop(name, None)
    return rows
