"""Compile the kernel library for sm_100a with nvcc and load it.

The library is plain CUDA C++ with ``extern "C"`` launchers (no Python or torch headers),
so a cold build takes well under a minute.  It is built in-tree, into ``csrc/_build``,
the first time it is needed and again whenever a source file or a flag changes; if the
package folder is not writable the build goes to a per-user folder under the system's
temporary directory.  Progress lines go to stderr while it compiles.
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libnimbus_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[nimbus-b200] {msg}", file=sys.stderr, flush=True)


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def find_nvcc() -> str:
    candidates = []
    for var in ("NVCC", "CUDACXX"):
        if os.environ.get(var):
            candidates.append(os.environ[var])
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(os.path.join(os.environ[var], "bin", "nvcc"))
    which = shutil.which("nvcc")
    if which:
        candidates.append(which)
    candidates += ["/usr/local/cuda/bin/nvcc", "/opt/cuda/bin/nvcc"]
    for c in candidates:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (set CUDA_HOME or NVCC); the kernel library cannot be built")


def source_hash() -> str:
    h = hashlib.sha256()
    for p in sources() + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe_{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("NIMBUS_B200_BUILD_DIR")
    if env:
        d = Path(env)
        if not _writable(d):
            raise BuildError(f"NIMBUS_B200_BUILD_DIR={env} is not writable")
        return d
    d = CSRC / "_build"
    if _writable(d):
        return d
    d = Path(tempfile.gettempdir()) / f"nimbus_b200_build_{os.getuid()}"
    if _writable(d):
        return d
    raise BuildError("no writable folder for the kernel library build")


def _run(cmd: list[str], what: str) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed (exit {proc.returncode}):\n{' '.join(cmd)}\n{proc.stdout}")
    warnings = [l for l in proc.stdout.splitlines() if "warning" in l.lower()]
    if warnings and os.environ.get("NIMBUS_B200_VERBOSE_BUILD"):
        _log(f"{what}: " + " | ".join(warnings[:5]))


def build(force: bool = False, verbose: bool = True) -> Path:
    """Make sure the library is built for the current sources; return its path."""
    with _lock:
        d = build_dir()
        lib = d / LIB_NAME
        stamp = d / "build.json"
        want = source_hash()
        if not force and lib.exists() and stamp.exists():
            try:
                if json.loads(stamp.read_text()).get("hash") == want:
                    return lib
            except (OSError, json.JSONDecodeError):
                pass
        nvcc = find_nvcc()
        srcs = sources()
        if not srcs:
            raise BuildError(f"no .cu sources in {CSRC}")
        t0 = time.time()
        if verbose:
            _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {d} (first call only)")
        obj_dir = d / "obj"
        obj_dir.mkdir(parents=True, exist_ok=True)
        stems = {src.stem for src in srcs}
        for old in obj_dir.glob("*.o"):            # objects whose source is gone
            if old.stem not in stems:
                old.unlink(missing_ok=True)

        done = threading.Event()

        def heartbeat():
            while not done.wait(10.0):
                _log(f"still compiling ... {time.time() - t0:.0f}s")

        hb = threading.Thread(target=heartbeat, daemon=True)
        if verbose:
            hb.start()

        def compile_one(src: Path) -> Path:
            obj = obj_dir / (src.stem + ".o")
            cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            _run(cmd, f"nvcc {src.name}")
            if verbose:
                _log(f"compiled {src.name} ({time.time() - t0:.0f}s)")
            return obj

        try:
            workers = max(1, min(len(srcs), os.cpu_count() or 4, 8))
            with ThreadPoolExecutor(workers) as pool:
                objs = list(pool.map(compile_one, srcs))
            tmp = d / (LIB_NAME + f".tmp{os.getpid()}")
            _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs)], "link")
            os.replace(tmp, lib)
            stamp.write_text(json.dumps({"hash": want, "nvcc": nvcc,
                                         "sources": [s.name for s in srcs]}))
        finally:
            done.set()
        if verbose:
            _log(f"built {lib.name} in {time.time() - t0:.0f}s")
        return lib


def load() -> ctypes.CDLL:
    """Build if needed, then load the library.  Raises if it cannot be built or loaded:
    there is no fallback path."""
    global _lib
    if _lib is not None:
        return _lib
    path = build()
    try:
        lib = ctypes.CDLL(str(path))
    except OSError as e:
        raise BuildError(f"cannot load {path}: {e}") from e
    _lib = lib
    return lib
