"""Compiles the CUDA sources of ``csrc/`` for sm_100a with nvcc and caches the shared
libraries.

Each library is keyed by a hash of its sources, the headers beside them (``*.cuh`` and
``*.h``) and its flags, so an
edited kernel is rebuilt and an unchanged one is loaded as is.  Libraries are kept in
``scratch_llm_b200/_build`` when that folder can be written, else in a per-user folder under
the system's temporary directory; no home directory is needed.  What a model needs is compiled
at its first use (the attention kernels once per head size), several files at a time, with a
progress line on stderr every few seconds.

The reference builds its kernels with ``setup.py``/CMake for sm_90a and sm_100a
(setup.py:45-135, CMakeLists.txt:71-129); here only sm_100a exists.
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
from typing import Iterable, Sequence

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
BASE_FLAGS = ("-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden")

_lock = threading.Lock()
_done: dict[str, Path] = {}


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").is_file():
            return str(Path(root) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc not found (looked in $CUDA_HOME, /usr/local/cuda and PATH): the "
                     "engine's CUDA kernels cannot be compiled, and there is no fallback")


_build_dir: Path | None = None


def build_dir() -> Path:
    global _build_dir
    with _lock:
        if _build_dir is None:
            _build_dir = _pick_build_dir()
        return _build_dir


def _pick_build_dir() -> Path:
    override = os.environ.get("SCRATCH_LLM_B200_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(Path(__file__).resolve().parent.parent / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"scratch_llm_b200_build_{os.getuid()}")
    for c in candidates:
        try:
            c.mkdir(parents=True, exist_ok=True)
            probe = c / f".w{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
            return c
        except OSError:
            continue
    raise BuildError("no writable folder for compiled kernels; set SCRATCH_LLM_B200_BUILD_DIR")


def _digest(sources: Sequence[Path], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for p in sorted([*CSRC.glob("*.cuh"), *CSRC.glob("*.h")]):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    for p in sources:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources: Sequence[str], defines: Iterable[str] = (),
                 extra_flags: Iterable[str] = ()) -> tuple[Path, list[str]]:
    srcs = [CSRC / s for s in sources]
    flags = [*BASE_FLAGS, *ARCH_FLAGS, *(f"-D{d}" for d in defines), *extra_flags]
    out = build_dir() / f"lib{name}_{_digest(srcs, flags)}.so"
    cmd = [find_nvcc(), *flags, f"-I{CSRC}", *map(str, srcs), "-o"]
    return out, cmd


def compile_library(name: str, sources: Sequence[str], defines: Iterable[str] = (),
                    extra_flags: Iterable[str] = (), verbose: bool = True) -> Path:
    """Return the path of the built library, compiling it first if it is not cached."""
    out, cmd = library_path(name, sources, defines, extra_flags)
    key = str(out)
    with _lock:
        if key in _done:
            return _done[key]
    if not out.is_file():
        if verbose:
            print(f"[scratch_llm_b200] compiling {name} for sm_100a ...", file=sys.stderr,
                  flush=True)
        tmp = out.with_suffix(f".tmp{os.getpid()}.{threading.get_ident()}.so")
        env = dict(os.environ)
        env.setdefault("TMPDIR", tempfile.gettempdir())
        proc = subprocess.run([*cmd, str(tmp)], capture_output=True, text=True, env=env)
        if proc.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise BuildError(f"nvcc failed for {name}:\n{' '.join(cmd)}\n{proc.stdout}\n"
                             f"{proc.stderr}")
        os.replace(tmp, out)
        # builds of earlier versions of this library's sources are of no more use
        prefix = out.name[:out.name.rfind("_") + 1]
        for old in out.parent.glob(prefix + "*.so"):
            if old != out and ".tmp" not in old.name:
                try:
                    old.unlink()
                except OSError:
                    pass
    with _lock:
        _done[key] = out
    return out


def compile_many(jobs: Sequence[tuple[str, Sequence[str], Sequence[str]]],
                 verbose: bool = True) -> list[Path]:
    """Compile several libraries at once: ``jobs`` are (name, sources, defines)."""
    todo = [j for j in jobs if not library_path(j[0], j[1], j[2])[0].is_file()]
    if not todo:
        return [compile_library(*j, verbose=False) for j in jobs]
    start = time.monotonic()
    if verbose:
        print(f"[scratch_llm_b200] first use: compiling {len(todo)} CUDA "
              f"librar{'y' if len(todo) == 1 else 'ies'} for sm_100a "
              f"({', '.join(j[0] for j in todo)})", file=sys.stderr, flush=True)
    with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1, 8)) as pool:
        futures = [pool.submit(compile_library, j[0], j[1], j[2], (), False) for j in jobs]
        while True:
            pending = [f for f in futures if not f.done()]
            if not pending:
                break
            time.sleep(0.25)
            if verbose and int(time.monotonic() - start) % 5 == 0 and \
                    (time.monotonic() - start) % 5 < 0.25:
                print(f"[scratch_llm_b200] ... still compiling, {len(pending)} to go "
                      f"({time.monotonic() - start:.0f} s)", file=sys.stderr, flush=True)
        paths = [f.result() for f in futures]
    if verbose:
        print(f"[scratch_llm_b200] compiled in {time.monotonic() - start:.1f} s",
              file=sys.stderr, flush=True)
    return paths
