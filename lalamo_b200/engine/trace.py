"""Trace replay: feeds given token ids through the engine step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: every step goes through
:meth:`lalamo_b200.engine.engine.Engine.step`, the function generation uses.

Input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the wanted
places (order of the entries and of ``want``) as little-endian float32 ``[wanted, vocab]``.  After
every step a line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import IO, Iterable

import numpy as np

from .engine import Engine, EngineConfig
from .executor import StepEntry

__all__ = ["TRACE_PAGE_SIZE", "replay", "run"]

TRACE_PAGE_SIZE = 16  # divides 64: a request's pages never cover more than its count rounded up to 64
MAX_LIVE_REQUESTS = 8


def replay(engine: Engine, lines: Iterable[str], out_dir: Path, reply: IO[str]) -> None:
    out_dir.mkdir(parents=True, exist_ok=True)
    live: set[str] = set()
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step_index = record["step"]
        entries = []
        for item in record.get("entries", []):
            request_id = str(item["id"])
            if request_id not in live:
                engine.admit(request_id)
                live.add(request_id)
            entries.append(StepEntry(request_id, [int(t) for t in item["tokens"]], [int(w) for w in item.get("want", [])]))
        logits = engine.step(entries)
        if logits.shape[0] > 0:
            host = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            host.tofile(out_dir / f"{step_index}.f32")
        for request_id in record.get("end", []):
            request_id = str(request_id)
            if request_id in live:
                engine.release(request_id)
                live.discard(request_id)
        engine.executor.check_status()
        reply.write(f"done {step_index}\n")
        reply.flush()


def run(model_dir: str, dtype: str, out_dir: str, max_tokens: int, poison_freed: bool = False) -> int:
    """``poison_freed`` overwrites pages and state slots with NaN when they are given back (a test
    option: logits must not change, since nothing may be read from memory a request does not hold)."""
    page = TRACE_PAGE_SIZE
    config = EngineConfig(
        dtype=dtype,
        page_size=page,
        max_tokens=-(-max_tokens // page) * page,
        max_requests=MAX_LIVE_REQUESTS,
        poison_freed=poison_freed,
    )
    engine = Engine.load(model_dir, config)
    replay(engine, sys.stdin, Path(out_dir), sys.stdout)
    return 0
