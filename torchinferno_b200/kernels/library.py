"""Build and load the engine's CUDA library (sm_100a only).

The kernels live in ``torchinferno_b200/csrc/*.cu`` behind a plain C interface
and are compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a`` into one
shared object, ``csrc/_build/libtorchinferno_b200.so``, at the first call that
needs them.  A stamp (hash of sources, headers, flags and compiler version)
beside the library decides whether it is current.  When the package folder is
not writable the build goes to a per-user folder under the system's temporary
directory.  There is no fallback: if the library cannot be built or loaded,
:func:`load_library` raises and nothing else in the engine runs.

The shape of the arrangement (native code prepared as an artifact, loaded by a
Python host) follows src/torchinferno/kernels/csrc/sgl_fp8_out.cpp:74-82 and its
loader in the reference.
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
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libtorchinferno_b200.so"
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
NVCC_FLAGS = ("-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr")

_lock = threading.Lock()
_library: ctypes.CDLL | None = None


class KernelBuildError(RuntimeError):
    pass


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def find_nvcc() -> str:
    for candidate in (os.environ.get("TORCHINFERNO_B200_NVCC"), shutil.which("nvcc"),
                      "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise KernelBuildError("nvcc not found: the CUDA kernels cannot be built (no fallback exists)")


def _nvcc_version(nvcc: str) -> str:
    out = subprocess.run([nvcc, "--version"], capture_output=True, text=True, check=False)
    return out.stdout.strip().splitlines()[-1] if out.stdout else "unknown"


def _stamp(nvcc: str) -> str:
    digest = hashlib.sha256()
    for path in _sources() + _headers():
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    digest.update(_nvcc_version(nvcc).encode())
    return digest.hexdigest()


def _flags() -> list[str]:
    return list(ARCH_FLAGS) + list(NVCC_FLAGS)


def _build_dirs() -> list[Path]:
    dirs = [CSRC / "_build"]
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(Path(tempfile.gettempdir()) / f"torchinferno_b200-{uid}" / "_build")
    return dirs


def _writable(directory: Path) -> bool:
    try:
        directory.mkdir(parents=True, exist_ok=True)
        probe = directory / f".probe-{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def _say(message: str, verbose: bool) -> None:
    if verbose:
        print(f"[torchinferno_b200] {message}", file=sys.stderr, flush=True)


def _current(directory: Path, stamp: str) -> bool:
    lib, mark = directory / LIB_NAME, directory / "stamp.txt"
    return lib.is_file() and mark.is_file() and mark.read_text().strip() == stamp


def build_library(verbose: bool = True, force: bool = False) -> Path:
    """Compile what is not current and return the path of the shared object."""
    sources = _sources()
    if not sources:
        raise KernelBuildError(f"no CUDA sources under {CSRC}")
    nvcc = find_nvcc()
    stamp = _stamp(nvcc)
    if not force:
        for directory in _build_dirs():
            if _current(directory, stamp):
                return directory / LIB_NAME
    directory = next((d for d in _build_dirs() if _writable(d)), None)
    if directory is None:
        raise KernelBuildError("no writable folder for the kernel build: tried "
                               + ", ".join(str(d) for d in _build_dirs()))
    _say(f"compiling {len(sources)} CUDA sources for sm_100a into {directory} (first call only)", verbose)
    started = time.time()
    flags = _flags()

    def compile_one(src: Path) -> Path:
        obj = directory / (src.stem + ".o")
        cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        t0 = time.time()
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
        _say(f"  compiled {src.name} in {time.time() - t0:.1f}s", verbose)
        return obj

    workers = max(1, min(len(sources), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        objects = list(pool.map(compile_one, sources))
    tmp_lib = directory / (LIB_NAME + f".tmp{os.getpid()}")
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *[str(o) for o in objects]]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, directory / LIB_NAME)
    (directory / "stamp.txt").write_text(stamp + "\n")
    _say(f"built {LIB_NAME} in {time.time() - started:.1f}s", verbose)
    return directory / LIB_NAME


def load_library(verbose: bool = True) -> ctypes.CDLL:
    """Return the loaded kernel library, building it first when needed."""
    global _library
    with _lock:
        if _library is None:
            path = build_library(verbose=verbose)
            try:
                _library = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelBuildError(f"cannot load {path}: {exc}") from exc
            _library._path = str(path)  # type: ignore[attr-defined]
        return _library


def library_path() -> str | None:
    return None if _library is None else getattr(_library, "_path", None)
