"""Compile the sm_100a kernels on first use and load them with ctypes.

Each ``.cu`` file becomes one shared object, built by ``nvcc`` into ``_build/``
beside the sources (or, when that folder cannot be written, into a folder under
the system's temporary directory) under a name that carries a hash of the source
text and the flags, so an edited source is rebuilt and a built one is reused.
Only what a run needs is compiled: a library is built when the first operation
that lives in it is called.  There is no fallback: if ``nvcc`` is missing or a
build fails, the operation raises.
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

SOURCE_DIR = Path(__file__).resolve().parent
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]
# Libraries and extra flags per source file.
EXTRA_FLAGS: dict[str, list[str]] = {
    "gemm_bf16": ["-lcuda"],
}
LIBRARIES = ("norm", "rope_cache", "attention_generic", "gemm_f32", "attention_bf16", "gemm_bf16",
             "sampling", "decode_attention_static")

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    found = shutil.which("nvcc")
    if found:
        return found
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").is_file():
            return str(Path(root) / "bin" / "nvcc")
    raise KernelBuildError(
        "nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda): the engine's kernels are compiled "
        "from source for sm_100a and there is no other code path")


def _flags(name: str) -> list[str]:
    return NVCC_FLAGS + EXTRA_FLAGS.get(name, [])


def _build_dir() -> Path:
    override = os.environ.get("B200_KERNEL_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(SOURCE_DIR / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"b200_kernels_{os.getuid()}")
    for folder in candidates:
        try:
            folder.mkdir(parents=True, exist_ok=True)
            probe = folder / f".write_probe_{os.getpid()}_{threading.get_ident()}"
            probe.write_text("")
            probe.unlink()
            return folder
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for built kernels among {candidates}")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update((SOURCE_DIR / f"{name}.cu").read_bytes())
    for header in sorted([*SOURCE_DIR.glob("*.cuh"), *SOURCE_DIR.glob("*.h")]):
        h.update(header.read_bytes())
    h.update(" ".join(_flags(name)).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> Path | None:
    """Path of the built library for the current sources, if it exists anywhere."""
    file_name = f"{name}-{_digest(name)}.so"
    for folder in (SOURCE_DIR / "_build", Path(tempfile.gettempdir()) / f"b200_kernels_{os.getuid()}"):
        if (folder / file_name).is_file():
            return folder / file_name
    override = os.environ.get("B200_KERNEL_BUILD_DIR")
    if override and (Path(override) / file_name).is_file():
        return Path(override) / file_name
    return None


def compile_library(name: str, verbose: bool = True) -> Path:
    source = SOURCE_DIR / f"{name}.cu"
    if not source.is_file():
        raise KernelBuildError(f"no kernel source {source}")
    existing = library_path(name)
    if existing is not None:
        return existing
    folder = _build_dir()
    target = folder / f"{name}-{_digest(name)}.so"
    scratch = folder / f".{name}-{os.getpid()}-{threading.get_ident()}.so"
    command = [_nvcc(), *_flags(name), "-I", str(SOURCE_DIR), "-o", str(scratch), str(source)]
    started = time.time()
    if verbose:
        print(f"[b200 kernels] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = process.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[b200 kernels] still compiling {name}.cu ({time.time() - started:.0f} s)",
                      file=sys.stderr, flush=True)
    if process.returncode != 0:
        scratch.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed on {source.name}:\n{' '.join(command)}\n{output}")
    os.replace(scratch, target)     # atomic: a concurrent builder sees either nothing or the whole file
    if verbose:
        print(f"[b200 kernels] built {target.name} in {time.time() - started:.1f} s",
              file=sys.stderr, flush=True)
    return target


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library ``name``; compiled first if its build is missing."""
    library = _loaded.get(name)
    if library is not None:
        return library
    with _lock:
        library = _loaded.get(name)
        if library is None:
            path = compile_library(name)
            library = ctypes.CDLL(str(path))
            library.b200_last_error.restype = ctypes.c_char_p
            _loaded[name] = library
    return library


def is_loaded(name: str) -> bool:
    """Whether this process has loaded the library (and so may have launched its kernels)."""
    return name in _loaded


def compile_all(verbose: bool = True) -> list[Path]:
    """Build every kernel library that has a source file (several at a time)."""
    from concurrent.futures import ThreadPoolExecutor
    names = [name for name in LIBRARIES if (SOURCE_DIR / f"{name}.cu").is_file()]
    with ThreadPoolExecutor(max_workers=min(8, len(names) or 1)) as pool:
        built = list(pool.map(lambda n: compile_library(n, verbose), names))
    # Libraries of earlier versions of the sources are of no use to anyone: drop them.
    current = {path.name for path in built}
    for path in {p.parent for p in built}:
        for stale in path.glob("*.so"):
            if stale.name not in current and stale.name.split("-")[0] in LIBRARIES:
                try:
                    stale.unlink()
                except OSError:
                    pass
    return built
