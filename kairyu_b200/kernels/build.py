"""Compiles the CUDA sources under ``csrc/`` for sm_100a and loads them with ctypes.

Each ``.cu`` file becomes one shared library, built the first time a function
from it is needed (so a model only pays for the kernels it uses) and rebuilt
when the source, a header or the flags change.  Libraries are kept in-tree
under ``csrc/_build/``; when that is not writable a per-user temporary folder
is used.  There is no fallback: without ``nvcc`` or without the library the
call raises.
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared"]

# name -> extra nvcc flags; every library the package can load is listed here,
# so that a full build knows them all.
LIBRARIES: dict[str, list[str]] = {
    "elementwise": [],
    "rope_kv": [],
    "attention_generic": [],
    "attention_mma": [],
    "attention_decode_static": [],
    "attention_decode_tma": [],
    "attention_prefill_tc5": [],
    "gemm_f32": [],
    "gemm_skinny": [],
    "gemm_tc5": [],
    "sampling": [],
}

_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for candidate in (
        os.environ.get("KAIRYU_B200_NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
    ):
        if candidate and os.path.exists(candidate):
            return candidate
    raise KernelBuildError(
        "nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels of "
        "kairyu_b200 cannot be built, and there is no other implementation to fall back on"
    )


def build_dir() -> Path:
    override = os.environ.get("KAIRYU_B200_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"kairyu_b200_build_{os.getuid()}")
    for path in candidates:
        try:
            path.mkdir(parents=True, exist_ok=True)
            probe = path / f".write_probe_{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
            return path
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {candidates}")


def _signature(name: str, flags: list[str]) -> str:
    digest = hashlib.sha256()
    digest.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + flags).encode())
    for path in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [CSRC / f"{name}.cu"]:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def _say(message: str) -> None:
    print(f"[kairyu_b200] {message}", file=sys.stderr, flush=True)


def library_path(name: str) -> Path:
    return build_dir() / f"libkb_{name}.so"


def compile_library(name: str, *, force: bool = False, verbose_ptxas: bool = False) -> Path:
    """Build ``csrc/<name>.cu`` if its library is missing or stale; return the path."""
    if name not in LIBRARIES:
        raise KernelBuildError(f"unknown kernel library {name!r}; known: {sorted(LIBRARIES)}")
    flags = LIBRARIES[name]
    source = CSRC / f"{name}.cu"
    if not source.exists():
        raise KernelBuildError(f"kernel source {source} is missing")
    out = library_path(name)
    stamp = out.with_suffix(".sig")
    signature = _signature(name, flags)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == signature:
        return out
    nvcc = _nvcc()
    tmp = out.with_name(f"{out.stem}.{os.getpid()}.tmp.so")
    command = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *flags, f"-I{CSRC}", "-o", str(tmp), str(source)]
    if verbose_ptxas:
        command[1:1] = ["-Xptxas", "-v"]
    _say(f"compiling {source.name} for sm_100a ...")
    started = time.time()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(10.0):
            _say(f"  still compiling {source.name} ({time.time() - started:.0f} s)")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    output, _ = process.communicate()
    done.set()
    if process.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {source.name}:\n{output}")
    if verbose_ptxas and output:
        print(output, file=sys.stderr)
    os.replace(tmp, out)
    stamp.write_text(signature)
    _say(f"built {out.name} in {time.time() - started:.1f} s")
    return out


def load_library(name: str) -> ctypes.CDLL:
    with _lock:
        if name in _loaded:
            return _loaded[name]
        path = compile_library(name)
        try:
            library = ctypes.CDLL(str(path))
        except OSError as error:
            raise KernelBuildError(f"cannot load {path}: {error}") from error
        _loaded[name] = library
        return library


def build_all(*, force: bool = False, verbose_ptxas: bool = False) -> list[Path]:
    """Compile every library (the build check; needs no GPU)."""
    return [compile_library(name, force=force, verbose_ptxas=verbose_ptxas) for name in LIBRARIES]
