"""Compiles the CUDA sources of this package for sm_100a at their first use and loads them.

Each kernel library is one shared object built straight with nvcc (no framework headers, so a
library compiles in seconds) and exports plain C launchers.  A library is compiled only when
something asks for it, with the `-D` definitions that caller needs (a head size, for instance), so
a model compiles what it uses and nothing else.  Objects are kept beside the sources in
`csrc/_build/` (or under the temporary directory when the package is read-only), named by a hash
of sources, definitions and flags.
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
from typing import Dict, Mapping, Sequence, Tuple

CSRC = Path(__file__).resolve().parent.parent / "csrc"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# no fast-math flag: exp, division and sqrt keep their IEEE-accurate forms
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC"]


class KernelBuildError(RuntimeError):
    pass


_loaded: Dict[str, ctypes.CDLL] = {}
_by_request: Dict[tuple, ctypes.CDLL] = {}
_lock = threading.Lock()


def _nvcc() -> str:
    candidates = [os.environ.get("MODELS_B200_NVCC"), shutil.which("nvcc")]
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home:
            candidates.append(str(Path(home) / "bin" / "nvcc"))
    for c in candidates:
        if c and Path(c).is_file():
            return c
    raise KernelBuildError(
        "nvcc was not found (looked at $MODELS_B200_NVCC, PATH, $CUDA_HOME, /usr/local/cuda); "
        "the CUDA kernels of models_b200 cannot be built and there is no other path")


def _build_dir() -> Path:
    override = os.environ.get("MODELS_B200_BUILD_DIR")
    preferred = Path(override) if override else CSRC / "_build"
    try:
        preferred.mkdir(parents=True, exist_ok=True)
        probe = preferred / f".writable-{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"models_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _hash(sources: Sequence[Path], defines: Mapping[str, object], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    for path in list(sources) + headers:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(list(flags)).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources: Sequence[str], defines: Mapping[str, object] | None = None,
                 extra_flags: Sequence[str] = ()) -> Tuple[Path, list]:
    defines = dict(defines or {})
    paths = [CSRC / s for s in sources]
    for p in paths:
        if not p.is_file():
            raise KernelBuildError(f"kernel source {p} is missing")
    flags = ARCH_FLAGS + COMMON_FLAGS + list(extra_flags) + [f"-D{k}={v}" for k, v in sorted(defines.items())]
    tag = "".join(f"-{k.lower()}{v}" for k, v in sorted(defines.items()))
    out = _build_dir() / f"lib{name}{tag}-{_hash(paths, defines, flags)}.so"
    return out, flags + ["-I", str(CSRC)] + [str(p) for p in paths]


def build_library(name: str, sources: Sequence[str], defines: Mapping[str, object] | None = None,
                  extra_flags: Sequence[str] = (), quiet: bool = False) -> Path:
    """Compiles if the object is not there yet; returns its path.  Needs no GPU."""
    out, args = library_path(name, sources, defines, extra_flags)
    if out.is_file():
        return out
    nvcc = _nvcc()
    lock_path = out.with_suffix(".lock")
    with open(lock_path, "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        try:
            if out.is_file():
                return out
            tmp = out.with_name(out.name + f".tmp{os.getpid()}")
            cmd = [nvcc] + args + ["-o", str(tmp)]
            label = out.stem
            started = time.time()
            if not quiet:
                print(f"[models_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
            process = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            done = threading.Event()

            def heartbeat():
                while not done.wait(10.0):
                    if not quiet:
                        print(f"[models_b200] still compiling {label} ({time.time() - started:.0f} s)",
                              file=sys.stderr, flush=True)

            beat = threading.Thread(target=heartbeat, daemon=True)
            beat.start()
            output, _ = process.communicate()
            done.set()
            if process.returncode != 0 or not tmp.is_file():
                raise KernelBuildError(f"nvcc failed for {label} (exit {process.returncode}):\n{' '.join(cmd)}\n{output}")
            os.replace(tmp, out)
            if not quiet:
                print(f"[models_b200] compiled {label} in {time.time() - started:.1f} s", file=sys.stderr, flush=True)
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)
    try:
        lock_path.unlink()
    except OSError:
        pass
    return out


def load_library(name: str, sources: Sequence[str], defines: Mapping[str, object] | None = None,
                 extra_flags: Sequence[str] = ()) -> ctypes.CDLL:
    """The loaded library (compiled first if needed).  Raises KernelBuildError; never falls back."""
    quick = (name, tuple(sources), tuple(sorted((defines or {}).items())), tuple(extra_flags))
    lib = _by_request.get(quick)  # the common case: no hashing of sources on the way to a launch
    if lib is not None:
        return lib
    out, _ = library_path(name, sources, defines, extra_flags)
    key = str(out)
    with _lock:
        if key in _loaded:
            _by_request[quick] = _loaded[key]
            return _loaded[key]
        path = build_library(name, sources, defines, extra_flags)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise KernelBuildError(f"cannot load {path}: {error}") from error
        lib.mb_last_error.restype = ctypes.c_char_p
        _loaded[key] = lib
        _by_request[quick] = lib
        return lib


def loaded_libraries():
    return sorted(_loaded)
