"""Compiles the CUDA sources under `csrc/` with nvcc into shared libraries, on demand.

A library is built the first time something asks for it, for sm_100a only, and is
kept beside the package under `_build/` (or, when that folder cannot be written,
under the system's temporary folder).  Its file name carries a hash of the sources,
headers, flags and macro definitions, so an edited source is rebuilt and an
unchanged one is loaded as is.  Only what is asked for is compiled: a float32
replay never builds the tensor-core kernels, and attention is built for the head
size of the model at hand.  While nvcc runs, a line is printed every few seconds.
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

CSRC = Path(__file__).resolve().parents[1] / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for candidate in (os.environ.get("SHRIKE_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise BuildError(
        "nvcc was not found (looked at $SHRIKE_B200_NVCC, PATH and /usr/local/cuda/bin); "
        "shrike_b200 compiles its sm_100a kernels at first use and cannot run without them"
    )


def build_dir() -> Path:
    override = os.environ.get("SHRIKE_B200_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC.parent / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"shrike_b200_build_{os.getuid()}")
    for folder in candidates:
        try:
            folder.mkdir(parents=True, exist_ok=True)
            probe = folder / f".write_probe_{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return folder
        except OSError:
            continue
    raise BuildError("no writable folder for compiled kernels; set SHRIKE_B200_BUILD_DIR")


def _digest(sources, defines, extra_flags) -> str:
    h = hashlib.sha256()
    for path in sorted(CSRC.glob("*.cuh")) + [CSRC / s for s in sources]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(repr((sorted(defines.items()), extra_flags, ARCH_FLAGS, BASE_FLAGS)).encode())
    return h.hexdigest()[:12]


def library_path(name: str, sources, defines=None, extra_flags=()) -> Path:
    return build_dir() / f"{name}-{_digest(sources, defines or {}, list(extra_flags))}.so"


def compile_library(name: str, sources, defines=None, extra_flags=(), verbose=True) -> Path:
    """Builds (if needed) and returns the path of the library."""
    defines = defines or {}
    target = library_path(name, sources, defines, extra_flags)
    if target.is_file():
        return target
    lock_path = target.parent / ".build.lock"
    with open(lock_path, "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        try:
            if target.is_file():
                return target
            nvcc = find_nvcc()
            scratch = target.with_suffix(f".tmp{os.getpid()}.so")
            command = [nvcc, *BASE_FLAGS, *ARCH_FLAGS, *extra_flags]
            command += [f"-D{key}={value}" for key, value in sorted(defines.items())]
            command += ["-o", str(scratch)] + [str(CSRC / s) for s in sources]
            started = time.time()
            if verbose:
                print(f"[shrike_b200] compiling {name} for sm_100a ...", file=sys.stderr, flush=True)
            process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            done = threading.Event()

            def heartbeat():
                while not done.wait(10.0):
                    print(f"[shrike_b200] still compiling {name} ({time.time() - started:.0f}s)",
                          file=sys.stderr, flush=True)

            beat = threading.Thread(target=heartbeat, daemon=True)
            if verbose:
                beat.start()
            output, _ = process.communicate()
            done.set()
            if process.returncode != 0:
                scratch.unlink(missing_ok=True)
                raise BuildError(f"nvcc failed for {name}:\n{' '.join(command)}\n{output}")
            os.replace(scratch, target)
            for stale in target.parent.glob(f"{name}-*.so"):   # older builds of the same library
                if stale != target and ".tmp" not in stale.name:
                    stale.unlink(missing_ok=True)
            if verbose:
                print(f"[shrike_b200] built {target.name} in {time.time() - started:.1f}s",
                      file=sys.stderr, flush=True)
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)
    return target


def load_library(name: str, sources, defines=None, extra_flags=()) -> ctypes.CDLL:
    key = f"{name}:{sorted((defines or {}).items())}"
    with _lock:
        if key not in _loaded:
            _loaded[key] = ctypes.CDLL(str(compile_library(name, sources, defines, extra_flags)))
        return _loaded[key]


# The libraries of this package.
CORE_SOURCES = ["elementwise.cu", "gemm_fp32.cu", "sampling.cu"]
ATTENTION_SOURCES = ["attention_generic.cu", "attention_bf16.cu", "attention_tcgen05.cu"]


def core_library() -> ctypes.CDLL:
    return load_library("shrike_core", CORE_SOURCES)


def attention_library(head_dim: int) -> ctypes.CDLL:
    return load_library(f"shrike_attention_d{head_dim}", ATTENTION_SOURCES, {"SHRIKE_HEAD_DIM": head_dim})


def tensor_core_gemm_library() -> ctypes.CDLL:
    return load_library("shrike_gemm_tcgen05", ["gemm_tcgen05.cu"])


def layer_program_library() -> ctypes.CDLL:
    return load_library("shrike_layer_program", ["layer_program.cu"])


def build_all(head_dims=(16, 32, 48, 64, 128, 256)) -> list[Path]:
    """Everything the package can load, for the usual head sizes."""
    built = [compile_library("shrike_core", CORE_SOURCES), compile_library("shrike_gemm_tcgen05", ["gemm_tcgen05.cu"]),
             compile_library("shrike_layer_program", ["layer_program.cu"])]
    for head_dim in head_dims:
        built.append(compile_library(f"shrike_attention_d{head_dim}", ATTENTION_SOURCES,
                                     {"SHRIKE_HEAD_DIM": head_dim}))
    return built
