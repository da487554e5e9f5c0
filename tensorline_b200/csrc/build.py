"""Compiling and loading the CUDA libraries.

The kernels are plain C-interface shared libraries built with nvcc for sm_100a and loaded with
ctypes; they take raw device pointers and a stream, so compiling them needs no framework headers
and takes seconds.  A library is built at its first use from the sources beside this file,
into `csrc/_build/` (or, if that is not writable, a per-user folder under the system temp
directory), under a name that carries a hash of its sources and flags: a changed source is a new
file, an unchanged one is never compiled twice.  Kernels whose tile shapes depend on the model
(attention on the head size) are compiled for the sizes this model has, nothing more.

There is no fallback: if nvcc or a source is missing, or compilation fails, `KernelBuildError`
is raised with the compiler's output.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC,-fvisibility=hidden"]

# The checking build: TENSORLINE_B200_CHECK=1 compiles every library with -DTL_CHECK=1 (bounds checks on every
# block-table and page index inside the kernels, see common.cuh); it is a library of its own beside the ordinary one.
CHECK_BUILD = os.environ.get("TENSORLINE_B200_CHECK", "0") == "1"
# The tracing build: TENSORLINE_B200_TRACE=1 compiles every library with -DTL_TRACE=1 (global-timer stamps in the kernels
# that wait on the kernel in front of them, see common.cuh and tensorline_b200/timeline.py) under a name of its own.
TRACE_BUILD = os.environ.get("TENSORLINE_B200_TRACE", "0") == "1"

_loaded: dict = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise KernelBuildError("nvcc was not found (PATH, $NVCC, /usr/local/cuda/bin): the CUDA kernels "
                           "of this engine cannot be built, and there is no other code path")


def build_dir() -> Path:
    env = os.environ.get("TENSORLINE_B200_BUILD_DIR")
    cands = [Path(env)] if env else []
    cands += [CSRC / "_build", Path(tempfile.gettempdir()) / f"tensorline_b200_build_{os.getuid()}"]
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".w{os.getpid()}_{threading.get_ident()}"      # several threads may build at once
            probe.write_bytes(b"")
            probe.unlink()
            return d
        except OSError:
            continue
    raise KernelBuildError("no writable folder for compiled kernels: tried " + ", ".join(map(str, cands)))


def _digest(sources, flags) -> str:
    h = hashlib.sha256()
    for f in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [CSRC / s for s in sources]:
        if not f.is_file():
            raise KernelBuildError(f"kernel source {f} is missing")
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources, defines: dict | None = None, extra_flags=(), check: bool | None = None,
                 trace: bool | None = None) -> tuple:
    """(path, flags, already built).  `check` / `trace`: the checking / tracing build of the library (None: as the
    environment says)."""
    check = CHECK_BUILD if check is None else check
    trace = TRACE_BUILD if trace is None else trace
    defines = dict(defines or {})
    if check:
        defines["TL_CHECK"] = 1
    if trace:
        defines["TL_TRACE"] = 1
    flags = ARCH_FLAGS + BASE_FLAGS + [f"-D{k}={v}" for k, v in sorted(defines.items())] + list(extra_flags)
    tag = _digest(sources, flags)
    if check:
        name = name + "_chk"
    if trace:
        name = name + "_trc"
    fname = f"lib{name}_{tag}.so"
    home = CSRC / "_build"
    if (home / fname).is_file():
        return home / fname, flags, True
    spare = Path(tempfile.gettempdir()) / f"tensorline_b200_build_{os.getuid()}" / fname
    if spare.is_file():
        # built while the package's own folder could not be written: move in beside the sources if that is possible
        # now (a copy of the package then carries its libraries along), else use it where it is
        try:
            home.mkdir(parents=True, exist_ok=True)
            tmp = home / f".{fname}.{os.getpid()}"
            shutil.copyfile(spare, tmp)
            os.replace(tmp, home / fname)
            return home / fname, flags, True
        except OSError:
            return spare, flags, True
    return build_dir() / fname, flags, False


def build_library(name: str, sources, defines: dict | None = None, extra_flags=(), verbose: bool = True,
                  check: bool | None = None, trace: bool | None = None) -> Path:
    """Compile (if not yet built) and return the path of the shared library."""
    path, flags, exists = library_path(name, sources, defines, extra_flags, check, trace)
    if exists:
        return path
    if CHECK_BUILD if check is None else check:
        name = name + "_chk"
    if TRACE_BUILD if trace is None else trace:
        name = name + "_trc"
    nvcc = _nvcc()
    tmp = path.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc] + flags + ["-I", str(CSRC), "-o", str(tmp)] + [str(CSRC / s) for s in sources]
    if verbose:
        print(f"[tensorline_b200] compiling {name} ({', '.join(sources)}) for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(15.0):
            print(f"[tensorline_b200]   still compiling {name}: {time.time() - t0:.0f} s", file=sys.stderr, flush=True)

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    try:
        env = dict(os.environ)
        env.setdefault("TMPDIR", str(path.parent))      # nvcc's intermediates beside the output
        proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    finally:
        done.set()
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed for {name}:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, path)                               # atomic: concurrent builders agree
    for old in path.parent.glob(f"lib{name}_*.so"):     # builds of this library from earlier sources
        if old != path and re.fullmatch(rf"lib{re.escape(name)}_[0-9a-f]{{16}}\.so", old.name):
            try:
                old.unlink()
            except OSError:
                pass                                    # another process may still have it mapped, or it is not ours
    if verbose:
        print(f"[tensorline_b200] built {path.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return path


def load_library(name: str, sources, defines: dict | None = None, extra_flags=()) -> ctypes.CDLL:
    key = (name, tuple(sources), tuple(sorted((defines or {}).items())), tuple(extra_flags))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = build_library(name, sources, defines, extra_flags)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _loaded[key] = lib
        return lib
