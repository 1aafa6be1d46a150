"""Drives ``bin/trace_run`` as a child process: sends steps, waits for ``done``, reads logits."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


class TraceRun:
    def __init__(self, model_dir: Path, dtype: str, out_dir: Path, max_tokens: int, vocab: int, poison_freed: bool = False) -> None:
        self.out_dir = Path(out_dir)
        self.vocab = vocab
        self.step_index = 0
        self.process = subprocess.Popen(
            [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir),
             "--max-tokens", str(max_tokens)] + (["--poison-freed"] if poison_freed else []),
            stdin=subprocess.PIPE,
            stdout=subprocess.PIPE,
            text=True,
            env={**os.environ, "PYTHONUNBUFFERED": "1"},
        )

    def step(self, entries: list[dict], end: list[str] = ()) -> np.ndarray | None:
        """Runs one step; returns the wanted logits [wanted, vocab] or None."""
        index = self.step_index
        self.step_index += 1
        record = {"step": index, "entries": entries, "end": list(end)}
        assert self.process.stdin is not None and self.process.stdout is not None
        self.process.stdin.write(json.dumps(record) + "\n")
        self.process.stdin.flush()
        line = self.process.stdout.readline()
        if line.strip() != f"done {index}":
            code = self.process.poll()
            raise RuntimeError(f"trace_run answered {line!r} (exit code {code}) to step {index}")
        wanted = sum(len(entry.get("want", [])) for entry in entries)
        if wanted == 0:
            return None
        data = np.fromfile(self.out_dir / f"{index}.f32", dtype="<f4")
        return data.reshape(wanted, self.vocab)

    def close(self) -> int:
        assert self.process.stdin is not None
        self.process.stdin.close()
        return self.process.wait(timeout=120)
