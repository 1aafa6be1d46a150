"""What `bench.py` promises without a GPU: more than one GPU is refused with one line and exit code
2; the reference arm prints one JSON line and exits with 0 whether or not the reference can be
imported; and `main` does not shadow a module it uses later (a function-local import makes the name
local for the whole function: the branch that does not import it then fails at its first use)."""

from __future__ import annotations

import importlib.util
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run(*arguments: str) -> subprocess.CompletedProcess:
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *arguments], cwd=ROOT, capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused():
    done = run("--gpus", "2", "--steps", "1", "--warmup", "1")
    assert done.returncode == 2
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_prints_one_json_line():
    done = run("--impl", "reference", "--gpus", "1", "--steps", "1", "--warmup", "1")
    assert done.returncode == 0
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference"
    assert "unavailable" in record or "value" in record


def test_main_shadows_no_module_it_uses():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    imported_at_top = {name for name, value in vars(module).items() if isinstance(value, type(sys))}
    shadowed = imported_at_top & set(module.main.__code__.co_varnames)
    assert not shadowed, f"main() makes {sorted(shadowed)} local, which the module imports at the top"
