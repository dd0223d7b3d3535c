"""Trace replay: feeds given token ids through a model step by step and writes logits. It samples nothing and has
no forward pass, cache or loader of its own: every step is one `Engine.step` call, the function generation uses.

Steps are JSON objects, one a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry gives a request's next tokens and the places among them whose logits are wanted; `end` lists requests
that are finished after the step (their cache room is given back). For a step that wants something the logits are
written to OUT/<step>.f32 as little-endian float32 [wanted, vocab], in the order of the entries and of `want`. After
every step `done <step>` is printed and flushed. `bin/trace_run` and `dllm-b200 replay` both call `run`.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Iterable


def run(model: str, dtype: str, out: str, max_tokens: int, device: str = "cuda:0",
        lines: Iterable[str] | None = None, report: IO[str] | None = None) -> int:
    """Replays the steps read from `lines` (default: standard input). `max_tokens`: the most tokens live requests
    hold at any time, each request's count rounded up to a multiple of 64; it sizes the cache exactly."""
    from .engine.engine import Engine

    lines = sys.stdin if lines is None else lines
    report = sys.stdout if report is None else report
    os.makedirs(out, exist_ok=True)
    pages = -(-int(max_tokens) // 64)
    engine = Engine.from_folder(model, dtype=dtype, device=device, max_tokens=pages * 64, max_length=pages * 64,
                                max_slots=pages)
    slots: dict[str, int] = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = record.get("entries", [])
        for entry in entries:
            if entry["id"] not in slots:
                slots[entry["id"]] = engine.open(1)[0]
        if entries:
            logits = engine.step([slots[e["id"]] for e in entries], [e["tokens"] for e in entries],
                                 [e.get("want", []) for e in entries])
            if logits is not None:
                values = logits.detach().cpu().numpy()  # (waits for the step)
                engine.check()  # a kernel that gave up is an error, not a file of logits
                values.astype("<f4", copy=False).tofile(os.path.join(out, f"{step}.f32"))
        ended = [slots.pop(name) for name in record.get("end", []) if name in slots]
        if ended:
            engine.close(ended)
        print(f"done {step}", file=report, flush=True)
    return 0
