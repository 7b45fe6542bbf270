"""Ways of cutting the same requests into steps, for the replay tests."""
from __future__ import annotations

from typing import Dict, List

import torch


def steps_whole(reqs: Dict[str, List[int]]):
    """Each request alone and whole, every position wanted."""
    steps = []
    for rid, toks in reqs.items():
        steps.append({"entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def steps_tail_decode(reqs, tail: int = 32):
    """Most of a request in one step, the last `tail` tokens one by one."""
    steps = []
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": toks[i:i + 1], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def steps_portions(reqs, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 41)):
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in reqs.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            steps.append({"entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
            at += n
            k += 1
        steps[-1]["end"] = [rid]
    return steps


def steps_mixed(reqs, max_live: int = 4, prefill_sizes=(11, 2, 24, 5), decode_tail: int = 12):
    """Up to max_live requests alive: portions of some beside single tokens of others.
    A request is fed in portions until `decode_tail` tokens remain, then token by token;
    new requests start as others end, so that their pages are used again."""
    pending = list(reqs.items())
    live = []          # [rid, toks, at, portion counter]
    steps = []
    tick = 0
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live.append([rid, toks, 0, len(live)])
            if len(live) >= 2 and tick % 2 == 0:
                break                      # stagger arrivals
        entries, ended = [], []
        for item in live:
            rid, toks, at, k = item
            if (tick + k) % 5 == 4 and len(live) > 1:
                continue                   # this request sits the step out
            remaining = len(toks) - at
            n = 1 if remaining <= decode_tail else min(prefill_sizes[(k + tick) % len(prefill_sizes)],
                                                       remaining - decode_tail)
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": list(range(n))})
            item[2] = at + n
            if item[2] == len(toks):
                ended.append(rid)
        live = [it for it in live if it[0] not in ended]
        if entries:
            steps.append({"entries": entries, "end": ended})
        tick += 1
    return steps


def run_steps(engine, steps):
    """Drive Engine.step; returns {request id: logits [len, vocab]} on the CPU."""
    from llm_b200.engine.engine import StepEntry
    rows = {}
    for st in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        logits = engine.step(entries).float().cpu()
        at = 0
        for e in st["entries"]:
            n = len(e["want"])
            rows.setdefault(e["id"], []).append(logits[at:at + n].clone())
            at += n
        for rid in st["end"]:
            engine.release(rid)
    return {rid: torch.cat(parts, dim=0) for rid, parts in rows.items()}
