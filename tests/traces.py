"""Builders of replay traces: the same requests cut into steps in different ways.

A trace is a list of steps ``{"step": n, "entries": [{"id", "tokens", "want"}], "end": []}``
(the format ``bin/trace_run`` reads).  ``labels(step)`` names, for every wanted row of a
step, the request and the absolute position it belongs to, so that any way of cutting can
be compared with the plain implementation's logits at the same positions.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np

Step = Dict[str, object]


def whole(requests: Dict[str, Sequence[int]]) -> List[Step]:
    """Each request alone and whole, every position wanted."""
    steps = []
    for index, (name, tokens) in enumerate(requests.items()):
        steps.append({"step": index, "end": [name],
                      "entries": [{"id": name, "tokens": list(tokens),
                                   "want": list(range(len(tokens)))}]})
    return steps


def tail_decoded(requests: Dict[str, Sequence[int]], tail: int = 32) -> List[Step]:
    """Most of each request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for name, tokens in requests.items():
        tokens = list(tokens)
        head = max(1, len(tokens) - tail)
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": name, "tokens": tokens[:head], "want": list(range(head))}]})
        for position in range(head, len(tokens)):
            steps.append({"step": len(steps), "end": [name] if position == len(tokens) - 1 else [],
                          "entries": [{"id": name, "tokens": [tokens[position]], "want": [0]}]})
        if head == len(tokens):
            steps[-1]["end"] = [name]
    return steps


PORTIONS = (7, 2, 13, 3, 2, 31, 5, 2, 64, 11, 2, 17)


def chunked(requests: Dict[str, Sequence[int]], portions: Sequence[int] = PORTIONS) -> List[Step]:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    for offset, (name, tokens) in enumerate(requests.items()):
        tokens = list(tokens)
        cursor = 0
        index = offset           # each request starts somewhere else in the size list
        while cursor < len(tokens):
            size = min(portions[index % len(portions)], len(tokens) - cursor)
            index += 1
            steps.append({"step": len(steps), "end": [name] if cursor + size == len(tokens) else [],
                          "entries": [{"id": name, "tokens": tokens[cursor:cursor + size],
                                       "want": list(range(size))}]})
            cursor += size
    return steps


def mixed(requests: Dict[str, Sequence[int]], max_live: int = 4, seed: int = 0,
          decode_tail: int = 12, chunk_choices: Sequence[int] = (2, 3, 5, 8, 16, 24)) -> List[Step]:
    """Up to ``max_live`` requests at a time: portions of some prompts beside single decoded
    tokens of others; a request may sit a step out; new requests start when one ends."""
    rng = np.random.default_rng(seed)
    pending = [(name, list(tokens)) for name, tokens in requests.items()]
    live: Dict[str, Dict[str, object]] = {}
    steps: List[Step] = []
    while pending or live:
        while pending and len(live) < max_live:
            name, tokens = pending.pop(0)
            live[name] = {"tokens": tokens, "cursor": 0}
        entries = []
        ended = []
        names = list(live)
        for name in names:
            state = live[name]
            tokens, cursor = state["tokens"], state["cursor"]
            if len(names) > 1 and rng.random() < 0.2:
                continue                                  # left out of this step
            remaining = len(tokens) - cursor
            if remaining <= decode_tail:
                size = 1                                  # decoding: one token per step
            else:
                size = int(min(rng.choice(chunk_choices), remaining - decode_tail))
            entries.append({"id": name, "tokens": tokens[cursor:cursor + size],
                            "want": list(range(size))})
            state["cursor"] = cursor + size
            if state["cursor"] == len(tokens):
                ended.append(name)
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": ended})
        for name in ended:
            del live[name]
    return steps


def labels(step: Step, positions: Dict[str, int]) -> List[Tuple[str, int]]:
    """(request, absolute position) of every wanted row of ``step``; ``positions`` holds the
    number of tokens each request has fed so far and is advanced."""
    rows = []
    for entry in step["entries"]:
        base = positions.get(entry["id"], 0)
        for place in entry["want"]:
            rows.append((entry["id"], base + place))
        positions[entry["id"]] = base + len(entry["tokens"])
    for name in step["end"]:
        positions.pop(name, None)
    return rows


def live_token_need(steps: List[Step], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: Dict[str, int] = {}
    worst = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        worst = max(worst, sum(-(-count // round_to) * round_to for count in held.values()))
        for name in step["end"]:
            held.pop(name, None)
    return worst
