"""Builds the CUDA library from ``csrc/`` with nvcc for sm_100a.

The library is built in-tree (``miniserve-llm-nv_b200/_build/``) at the first call
that needs it and is rebuilt when a source or a flag changed (a digest of both is kept
beside it).  If that folder cannot be written, a per-user folder under the system's
temporary directory is used instead.  Each source file becomes one object file; they
are compiled in parallel and a progress line is printed every few seconds, because a
first build takes the better part of a minute.

The sources include no framework headers: they export plain C functions over raw device
pointers, so the build needs nvcc and a host compiler and nothing else.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent.parent
SOURCE_DIR = PACKAGE_DIR / "csrc"
LIBRARY_NAME = "libminiserve_b200_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


class KernelBuildError(RuntimeError):
    """nvcc is missing or a source failed to compile; the message carries the compiler's output."""


def find_nvcc() -> str:
    candidates = []
    for variable in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(variable):
            candidates.append(Path(os.environ[variable]) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        candidates.append(Path(found))
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    for candidate in candidates:
        if candidate.is_file():
            return str(candidate)
    raise KernelBuildError(
        "nvcc not found (looked at $CUDA_HOME/bin, $PATH and /usr/local/cuda/bin); "
        "the engine has no path without its CUDA library")


def source_files() -> list[Path]:
    return sorted(SOURCE_DIR.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for path in sorted(p for pattern in ("*.cu", "*.cuh", "*.h") for p in SOURCE_DIR.glob(pattern)):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()


def exported_signatures() -> dict:
    """``{name: (return kind, [argument kinds])}`` of every ``MS_EXPORT`` function in the sources, read from their
    prototypes: kinds are ``"pointer"`` (any pointer, and streams), ``"int"``, ``"float"``, ``"longlong"``,
    ``"string"`` (``const char*`` results) and ``"void"``.  The bindings give these to ctypes, so that calls pass
    plain Python numbers instead of building a ctypes object per argument."""
    import re

    def kind(text: str, result: bool = False) -> str:
        text = " ".join(text.split())
        if result and text.startswith("const char"):
            return "string"
        if "*" in text or "cudaStream_t" in text:
            return "pointer"
        if text.startswith("long long") or " long long" in text:
            return "longlong"
        if text.startswith("float") or text.startswith("const float"):
            return "float"
        if text.startswith("void"):
            return "void"
        if text.startswith("int") or text.startswith("const int") or text.startswith("unsigned"):
            return "int"
        raise KernelBuildError(f"cannot tell the ctypes kind of {text!r} in an exported prototype")

    found: dict = {}
    pattern = re.compile(r"MS_EXPORT\s+([\w\s\*]+?)\s*\b(ms_\w+)\s*\(([^)]*)\)", re.DOTALL)
    for path in source_files():
        for result, name, arguments in pattern.findall(path.read_text()):
            arguments = [a for a in (part.strip() for part in arguments.split(",")) if a and a != "void"]
            found[name] = (kind(result, result=True), [kind(a) for a in arguments])
    return found


def _build_dir() -> Path:
    in_tree = PACKAGE_DIR / "_build"
    try:
        in_tree.mkdir(exist_ok=True)
        probe = in_tree / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return in_tree
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"miniserve_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _say(message: str) -> None:
    print(f"[miniserve_b200] {message}", file=sys.stderr, flush=True)


def library_path(verbose: bool = True) -> Path:
    """Path of an up-to-date library, building it first if needed."""
    build_dir = _build_dir()
    library = build_dir / LIBRARY_NAME
    stamp = build_dir / (LIBRARY_NAME + ".sha256")
    digest = _digest()
    if library.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
        return library

    nvcc = find_nvcc()
    sources = source_files()
    if not sources:
        raise KernelBuildError(f"no CUDA sources under {SOURCE_DIR}")
    work = build_dir / f"obj_{digest[:12]}_{os.getpid()}"
    work.mkdir(parents=True, exist_ok=True)
    started = time.time()
    if verbose:
        _say(f"building {LIBRARY_NAME} from {len(sources)} CUDA sources for sm_100a (first use; about a minute)")

    done: list[str] = []
    lock = threading.Lock()

    def compile_one(source: Path) -> Path:
        obj = work / (source.stem + ".o")
        command = [nvcc, *NVCC_FLAGS, "-I", str(SOURCE_DIR), "-c", str(source), "-o", str(obj)]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {source.name}:\n{result.stdout}\n{result.stderr}")
        with lock:
            done.append(source.name)
        return obj

    stop = threading.Event()

    def progress() -> None:
        while not stop.wait(5.0):
            with lock:
                finished = len(done)
            _say(f"  compiling... {finished}/{len(sources)} files done, {time.time() - started:.0f} s")

    ticker = threading.Thread(target=progress, daemon=True)
    if verbose:
        ticker.start()
    try:
        with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 4)) as pool:
            objects = list(pool.map(compile_one, sources))
        temporary = build_dir / f".{LIBRARY_NAME}.{os.getpid()}"
        command = [nvcc, "-shared", "-o", str(temporary), *[str(o) for o in objects],
                   "-gencode", "arch=compute_100a,code=sm_100a"]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise KernelBuildError(f"linking {LIBRARY_NAME} failed:\n{result.stdout}\n{result.stderr}")
        os.replace(temporary, library)
        stamp.write_text(digest)
    finally:
        stop.set()
        shutil.rmtree(work, ignore_errors=True)
    if verbose:
        _say(f"built {library} in {time.time() - started:.0f} s")
    return library
