"""Builds and loads the CUDA extension (the ``.cu`` files under ``csrc/``).

The extension is one shared library of ``extern "C"`` launchers, compiled with ``nvcc`` for
sm_100a and loaded with ``ctypes``; launchers take raw device pointers and a stream.  It is built
in-tree (``lalamo_b200/_native/``) when that folder can be written, otherwise under the
temporary directory, and rebuilt when a source file changes.  There is no fallback: if the
library cannot be built or loaded, :func:`library` raises.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

__all__ = ["NativeBuildError", "build", "library", "library_path", "source_files"]

_SOURCE_DIR = Path(__file__).resolve().parent / "csrc"
_LIBRARY_NAME = "liblalamo_b200_kernels.so"
_NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "--shared",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]

_lock = threading.Lock()
_library: ctypes.CDLL | None = None


class NativeBuildError(RuntimeError):
    pass


def source_files() -> list[Path]:
    return sorted(_SOURCE_DIR.glob("*.cu"))


def _source_digest() -> str:
    digest = hashlib.sha256()
    for path in sorted(_SOURCE_DIR.glob("*.cu*")):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(_NVCC_FLAGS).encode())
    return digest.hexdigest()[:16]


def _find_nvcc() -> str:
    candidates = [
        os.environ.get("LALAMO_B200_NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ]
    for candidate in candidates:
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise NativeBuildError("nvcc was not found (looked at $LALAMO_B200_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin)")


def _build_dirs() -> list[Path]:
    dirs = [Path(__file__).resolve().parent / "_native"]
    user = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(Path(tempfile.gettempdir()) / f"lalamo_b200_native_{user}")
    return dirs


def _usable(directory: Path) -> bool:
    try:
        directory.mkdir(parents=True, exist_ok=True)
        probe = directory / f".probe_{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def library_path() -> Path | None:
    """The up-to-date built library, if there is one."""
    digest = _source_digest()
    for directory in _build_dirs():
        candidate = directory / _LIBRARY_NAME
        stamp = directory / "source.digest"
        if candidate.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
            return candidate
    return None


def build(verbose: bool = True, force: bool = False) -> Path:
    """Compiles every kernel for sm_100a; returns the library's path."""
    existing = None if force else library_path()
    if existing is not None:
        return existing
    nvcc = _find_nvcc()
    directory = next((d for d in _build_dirs() if _usable(d)), None)
    if directory is None:
        raise NativeBuildError(f"none of {[str(d) for d in _build_dirs()]} can be written")
    sources = source_files()
    objects: list[Path] = []
    started = time.time()
    processes: list[tuple[Path, subprocess.Popen]] = []
    compile_flags = [flag for flag in _NVCC_FLAGS if flag != "--shared"]
    for source in sources:
        target = directory / (source.stem + f".{os.getpid()}.o")
        objects.append(target)
        command = [nvcc, *compile_flags, "-c", str(source), "-o", str(target)]
        processes.append((source, subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    if verbose:
        print(f"[lalamo_b200] compiling {len(sources)} CUDA sources for sm_100a into {directory} ...", file=sys.stderr, flush=True)
    for source, process in processes:
        while True:
            try:
                output, _ = process.communicate(timeout=20)
                break
            except subprocess.TimeoutExpired:
                if verbose:
                    print(f"[lalamo_b200] still compiling ({source.name}, {time.time() - started:.0f} s) ...", file=sys.stderr, flush=True)
        if process.returncode != 0:
            for _, other in processes:
                if other.poll() is None:
                    other.kill()
            raise NativeBuildError(f"nvcc failed on {source.name}:\n{output}")
    temporary = directory / f"{_LIBRARY_NAME}.{os.getpid()}.tmp"
    link = subprocess.run(
        [nvcc, "--shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(temporary), *map(str, objects)],
        stdout=subprocess.PIPE,
        stderr=subprocess.STDOUT,
        text=True,
    )
    for target in objects:
        target.unlink(missing_ok=True)
    if link.returncode != 0:
        raise NativeBuildError(f"linking the kernel library failed:\n{link.stdout}")
    os.replace(temporary, directory / _LIBRARY_NAME)
    (directory / "source.digest").write_text(_source_digest())
    if verbose:
        print(f"[lalamo_b200] built {_LIBRARY_NAME} in {time.time() - started:.0f} s", file=sys.stderr, flush=True)
    return directory / _LIBRARY_NAME


def library() -> ctypes.CDLL:
    """The loaded kernel library (built at the first call if needed)."""
    global _library
    with _lock:
        if _library is None:
            path = build()
            try:
                _library = ctypes.CDLL(str(path))
            except OSError as error:
                raise NativeBuildError(f"cannot load {path}: {error}") from error
        return _library
