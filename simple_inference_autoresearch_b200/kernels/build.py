"""Compiles the CUDA units under ``csrc/`` for sm_100a with nvcc and loads them.

Each ``csrc/<unit>.cu`` becomes one shared object ``csrc/_build/libsiar_<unit>.so``
holding ``extern "C"`` launchers that take raw device pointers and a stream; they
are loaded with ctypes, so building needs nothing but nvcc (no Python or torch
headers) and takes seconds per unit.  A unit is compiled the first time something
asks for it, and again whenever its source, a header or the flags change.  There
is no fallback: a missing compiler or a failed build raises ``ExtensionError``.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path
from typing import Dict, Iterable, List

CSRC = Path(__file__).resolve().parent.parent / "csrc"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]

#: extra nvcc flags for profiling builds, e.g. SIAR_NVCC_FLAGS="-DSIAR_TIMING" compiles the
#: globaltimer stamps into the product and attention kernels (separate build folder per flag set)
EXTRA_FLAGS = os.environ.get("SIAR_NVCC_FLAGS", "").split()

#: every unit of the library, in the order ``build_all`` compiles them
ALL_UNITS = ("elementwise", "gemm_simt", "attention", "attention_mma", "attention_tc", "sampling", "gemm_tc")


class ExtensionError(RuntimeError):
    """The CUDA extension could not be built or loaded."""


_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _say(msg: str) -> None:
    print(f"[simple_inference_autoresearch_b200] {msg}", file=sys.stderr, flush=True)


def available_units() -> List[str]:
    return [u for u in ALL_UNITS if (CSRC / f"{u}.cu").exists()]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise ExtensionError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                         "the CUDA kernels cannot be built and there is no fallback")


def _build_dir() -> Path:
    """In-tree ``csrc/_build`` when it can be written, else a per-user temp folder."""
    d = CSRC / ("_build" if not EXTRA_FLAGS else "_build_" + hashlib.sha256(" ".join(EXTRA_FLAGS).encode()).hexdigest()[:8])
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.touch()
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"siar_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _fingerprint(unit: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + EXTRA_FLAGS).encode())
    for p in [CSRC / f"{unit}.cu"] + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _compile(unit: str, out: Path) -> None:
    src = CSRC / f"{unit}.cu"
    if not src.exists():
        raise ExtensionError(f"no such CUDA unit: {src}")
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [_nvcc(), *NVCC_FLAGS, *EXTRA_FLAGS, "-I", str(CSRC), "-o", str(tmp), str(src)]
    _say(f"compiling {src.name} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"  still compiling {src.name} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        output, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise ExtensionError(f"nvcc failed on {src.name} (exit {proc.returncode}):\n{output}")
    os.replace(tmp, out)
    _say(f"compiled {src.name} in {time.time() - t0:.1f} s")


def ensure_built(units: Iterable[str]) -> Dict[str, Path]:
    """Compile whatever of ``units`` is missing or stale; returns unit -> .so path."""
    bdir = _build_dir()
    result: Dict[str, Path] = {}
    todo = []
    for unit in units:
        so = bdir / f"libsiar_{unit}.so"
        stamp = bdir / f"libsiar_{unit}.hash"
        fp = _fingerprint(unit)
        result[unit] = so
        if not (so.exists() and stamp.exists() and stamp.read_text().strip() == fp):
            todo.append((unit, so, stamp, fp))
    if not todo:
        return result
    with open(bdir / ".lock", "w") as lockf:
        fcntl.flock(lockf, fcntl.LOCK_EX)  # another process may be building the same units
        try:
            errors: List[BaseException] = []

            def work(item):
                unit, so, stamp, fp = item
                try:
                    if so.exists() and stamp.exists() and stamp.read_text().strip() == fp:
                        return
                    _compile(unit, so)
                    stamp.write_text(fp)
                except BaseException as e:  # noqa: BLE001 - re-raised below
                    errors.append(e)

            threads = [threading.Thread(target=work, args=(it,)) for it in todo]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
            if errors:
                raise errors[0]
        finally:
            fcntl.flock(lockf, fcntl.LOCK_UN)
    return result


def load_unit(unit: str) -> ctypes.CDLL:
    """The loaded shared object of a unit (built first if needed)."""
    lib = _loaded.get(unit)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(unit)
        if lib is None:
            path = ensure_built([unit])[unit]
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise ExtensionError(f"cannot load {path}: {e}") from e
            _loaded[unit] = lib
    return lib


def build_all() -> Dict[str, Path]:
    return ensure_built(available_units())
